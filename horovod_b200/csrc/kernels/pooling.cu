// 3x3 / stride 2 / padding 1 max pooling on channels-last 16-bit activations
// (the ResNet stem), forward and backward.
//
// Forward: one thread owns 8 channels (16 bytes) of one output pixel, reads
// the up to nine input vectors of its window (neighbouring windows overlap, so
// most of them come from L1/L2), and writes the maxima plus one byte per
// channel that says which of the nine window positions won. Backward: one
// thread owns 8 channels of one INPUT pixel, looks at the up to four windows
// that cover it and adds the output gradients of those that picked this
// position: a gather, so no atomics and every byte of dx is written once.
// Both passes touch each byte of the big tensors once: forward reads x and
// writes y + y/2 bytes of indices, backward reads dy + indices and writes dx.
//
// Ties go to the first maximum in scan order (rows, then columns) and NaN
// wins over everything, which is the rule of PyTorch's max_pool2d, so the
// gradients agree with it element for element.
//
// The reference has no counterpart (it takes pooling from the framework).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"

namespace hvd {
namespace kern {

namespace {

template <typename T> __device__ __forceinline__ float pool_to_float(T v);
template <> __device__ __forceinline__ float pool_to_float(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float pool_to_float(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T pool_from_float(float v);
template <> __device__ __forceinline__ __half pool_from_float(float v) {
  return __float2half_rn(v);
}
template <> __device__ __forceinline__ __nv_bfloat16 pool_from_float(float v) {
  return __float2bfloat16_rn(v);
}

template <typename T> union Vec8 {
  uint4 raw;
  T e[8];
};
union Idx8 {
  uint2 raw;
  unsigned char e[8];
};

// I: type of the flat vector index. Tensors of fewer than 2^31 vectors (every
// practical activation) use 32-bit index arithmetic: the three divisions per
// thread cost several times the pooling itself when done in 64 bits.
template <typename T, typename I>
__global__ void __launch_bounds__(256)
maxpool3s2_forward_kernel(const T* __restrict__ x, T* __restrict__ y,
                          unsigned char* __restrict__ idx, int N, int H, int W, int C8, int Ho,
                          int Wo) {
  const I total = static_cast<I>(N) * Ho * Wo * C8;
  for (I t = blockIdx.x * static_cast<I>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<I>(gridDim.x) * blockDim.x) {
    const int c8 = static_cast<int>(t % C8);
    I r = t / C8;
    const int ow = static_cast<int>(r % Wo);
    r /= Wo;
    const int oh = static_cast<int>(r % Ho);
    const int n = static_cast<int>(r / Ho);
    const int h0 = oh * 2 - 1, w0 = ow * 2 - 1;
    float best[8];
    unsigned char arg[8];
    bool seen = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) best[i] = -INFINITY;
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
      const int h = h0 + kh;
      if (h < 0 || h >= H) continue;
#pragma unroll
      for (int kw = 0; kw < 3; ++kw) {
        const int w = w0 + kw;
        if (w < 0 || w >= W) continue;
        Vec8<T> v;
        v.raw = __ldg(reinterpret_cast<const uint4*>(x) +
                      ((static_cast<I>(n) * H + h) * W + w) * C8 + c8);
        const unsigned char pos = static_cast<unsigned char>(kh * 3 + kw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float f = pool_to_float(v.e[i]);
          // A NaN maximum stays (every comparison with it is false) unless a
          // later NaN replaces it, as in PyTorch.
          if (!seen || f > best[i] || f != f) {
            best[i] = f;
            arg[i] = pos;
          }
        }
        seen = true;
      }
    }
    Vec8<T> out;
    Idx8 oi;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      out.e[i] = pool_from_float<T>(best[i]);
      oi.e[i] = arg[i];
    }
    reinterpret_cast<uint4*>(y)[t] = out.raw;
    reinterpret_cast<uint2*>(idx)[t] = oi.raw;
  }
}

template <typename T, typename I>
__global__ void __launch_bounds__(256)
maxpool3s2_backward_kernel(const T* __restrict__ dy, const unsigned char* __restrict__ idx,
                           T* __restrict__ dx, int N, int H, int W, int C8, int Ho, int Wo) {
  const I total = static_cast<I>(N) * H * W * C8;
  for (I t = blockIdx.x * static_cast<I>(blockDim.x) + threadIdx.x; t < total;
       t += static_cast<I>(gridDim.x) * blockDim.x) {
    const int c8 = static_cast<int>(t % C8);
    I r = t / C8;
    const int w = static_cast<int>(r % W);
    r /= W;
    const int h = static_cast<int>(r % H);
    const int n = static_cast<int>(r / H);
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    // Windows oh with 2 oh - 1 <= h <= 2 oh + 1.
    const int oh_lo = h >> 1, oh_hi = (h + 1) >> 1;
    const int ow_lo = w >> 1, ow_hi = (w + 1) >> 1;
    for (int oh = oh_lo; oh <= oh_hi; ++oh) {
      if (oh >= Ho) continue;
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        if (ow >= Wo) continue;
        const unsigned char pos =
            static_cast<unsigned char>((h - (oh * 2 - 1)) * 3 + (w - (ow * 2 - 1)));
        const I o = ((static_cast<I>(n) * Ho + oh) * Wo + ow) * C8 + c8;
        Idx8 oi;
        oi.raw = __ldg(reinterpret_cast<const uint2*>(idx) + o);
        Vec8<T> g;
        g.raw = __ldg(reinterpret_cast<const uint4*>(dy) + o);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (oi.e[i] == pos) acc[i] += pool_to_float(g.e[i]);
      }
    }
    Vec8<T> out;
#pragma unroll
    for (int i = 0; i < 8; ++i) out.e[i] = pool_from_float<T>(acc[i]);
    reinterpret_cast<uint4*>(dx)[t] = out.raw;
  }
}

int GridFor(long long total) {
  const long long blocks = (total + 255) / 256;
  return static_cast<int>(blocks < 148 * 32 ? (blocks < 1 ? 1 : blocks) : 148 * 32);
}

// Whether every vector index of the larger tensor, plus one grid stride, fits
// a 32-bit int.
bool Fits32(long long input_vectors) {
  return input_vectors + 148LL * 32 * 256 < (1LL << 31);
}

}  // namespace

bool MaxPool3s2Supported(int channels) { return channels > 0 && channels % 8 == 0; }

cudaError_t LaunchMaxPool3s2Forward(const void* x, void* y, unsigned char* idx, int n, int h,
                                    int w, int channels, bool bf16, cudaStream_t stream) {
  if (!MaxPool3s2Supported(channels)) return cudaErrorInvalidValue;
  const int ho = (h + 2 - 3) / 2 + 1, wo = (w + 2 - 3) / 2 + 1;
  const long long total = static_cast<long long>(n) * ho * wo * (channels / 8);
  if (total == 0) return cudaSuccess;
  CountKernelLaunches(1);
  const bool small = Fits32(static_cast<long long>(n) * h * w * (channels / 8));
#define HVD_POOL_FWD(T, I)                                                                   \
  maxpool3s2_forward_kernel<T, I><<<GridFor(total), 256, 0, stream>>>(                       \
      static_cast<const T*>(x), static_cast<T*>(y), idx, n, h, w, channels / 8, ho, wo)
  if (bf16) {
    if (small) HVD_POOL_FWD(__nv_bfloat16, int); else HVD_POOL_FWD(__nv_bfloat16, long long);
  } else {
    if (small) HVD_POOL_FWD(__half, int); else HVD_POOL_FWD(__half, long long);
  }
#undef HVD_POOL_FWD
  return cudaGetLastError();
}

cudaError_t LaunchMaxPool3s2Backward(const void* dy, const unsigned char* idx, void* dx, int n,
                                     int h, int w, int channels, bool bf16,
                                     cudaStream_t stream) {
  if (!MaxPool3s2Supported(channels)) return cudaErrorInvalidValue;
  const int ho = (h + 2 - 3) / 2 + 1, wo = (w + 2 - 3) / 2 + 1;
  const long long total = static_cast<long long>(n) * h * w * (channels / 8);
  if (total == 0) return cudaSuccess;
  CountKernelLaunches(1);
  const bool small = Fits32(total);
#define HVD_POOL_BWD(T, I)                                                                   \
  maxpool3s2_backward_kernel<T, I><<<GridFor(total), 256, 0, stream>>>(                      \
      static_cast<const T*>(dy), idx, static_cast<T*>(dx), n, h, w, channels / 8, ho, wo)
  if (bf16) {
    if (small) HVD_POOL_BWD(__nv_bfloat16, int); else HVD_POOL_BWD(__nv_bfloat16, long long);
  } else {
    if (small) HVD_POOL_BWD(__half, int); else HVD_POOL_BWD(__half, long long);
  }
#undef HVD_POOL_BWD
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace hvd
