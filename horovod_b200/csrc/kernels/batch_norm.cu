// Training-mode batch normalisation for channels-last (NHWC) 16-bit
// activations, fused with what surrounds it in a residual network:
//   forward : statistics -> y = relu(x * scale + shift [+ residual])
//   backward: dz = dy * (y > 0); per-channel sum(dz), sum(dz * xhat);
//             dx = scale * (dz - sum(dz)/M - xhat * sum(dz*xhat)/M); dres = dz
// The tensor is treated as a row-major [M = N*H*W, C] matrix. A thread owns 8
// consecutive channels (one 16-byte access per row), a warp covers 256
// consecutive channels of one row (or several rows when C is smaller), so every
// access is a fully coalesced 512-byte line. Each pass is bound by HBM traffic:
// the forward reads x twice and writes y once (the PyTorch eager sequence
// batch_norm + add + relu makes eight passes), the backward reads dy, y, x
// twice and writes dx (and dres).
//
// Per-channel sums are accumulated in fp32 per thread (a few dozen rows), in
// fp32 across the CTA, and in fp64 across CTAs (atomicAdd on doubles), then
// mean/variance are formed in fp64.
//
// The reference has no counterpart: it takes batch normalisation from the
// framework (horovod/torch/sync_batch_norm.py:98-199 calls
// torch.batch_norm_stats / batch_norm_elemt / batch_norm_backward_reduce).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.h"

namespace hvd {
namespace kern {

namespace {

constexpr int BN_THREADS = 256;
// Resident CTAs per SM the compiler must leave room for (register budget):
// these are streaming kernels whose throughput is set by the bytes in flight
// per SM, i.e. by occupancy.
constexpr int BN_MIN_BLOCKS_APPLY = 3;   // <= 85 registers per thread
constexpr int BN_MIN_BLOCKS_REDUCE = 4;  // <= 64 registers per thread
constexpr int VEC = 8;  // 16-bit elements per 16-byte access

template <typename T> __device__ __forceinline__ float bn_to_float(T v);
template <> __device__ __forceinline__ float bn_to_float(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <> __device__ __forceinline__ float bn_to_float(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T bn_from_float(float v);
template <> __device__ __forceinline__ __nv_bfloat16 bn_from_float(float v) {
  return __float2bfloat16(v);
}
template <> __device__ __forceinline__ __half bn_from_float(float v) { return __float2half(v); }

template <typename T> union Vec8 {
  uint4 raw;
  T e[VEC];
};

__device__ __forceinline__ uint4 ldg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void stg16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}

// Thread geometry shared by all four kernels.
struct Tile {
  int txg;        // channel groups (of 8 channels) per CTA along x: min(C/8, 32)
  int ty;         // rows handled in parallel by a CTA: BN_THREADS / txg
  int tx, row;    // this thread's position
  int64_t group;  // global channel group of this thread
  __device__ __forceinline__ Tile(int C) {
    const int cg = C / VEC;
    txg = cg < 32 ? cg : 32;
    ty = BN_THREADS / txg;
    tx = threadIdx.x % txg;
    row = threadIdx.x / txg;
    group = static_cast<int64_t>(blockIdx.x) * txg + tx;
  }
};

// Rows [r0, r1) of this CTA.
__device__ __forceinline__ void cta_rows(int64_t M, int64_t* r0, int64_t* r1) {
  const int64_t per = (M + gridDim.y - 1) / gridDim.y;
  *r0 = blockIdx.y * per;
  *r1 = min(*r0 + per, M);
}

// Sums `acc` (NV values per thread) over the threads of the CTA that own the
// same channel group and adds the totals to the fp64 accumulators.
template <int NV>
__device__ __forceinline__ void reduce_to_global(const Tile& t, float (&acc)[NV][VEC],
                                                 double* const (&dst)[NV], int C) {
  __shared__ float red[BN_THREADS][NV * VEC + 1];
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int i = 0; i < VEC; ++i) red[threadIdx.x][k * VEC + i] = acc[k][i];
  __syncthreads();
  // One thread per (channel group, value): NV * VEC * txg <= 2 * 8 * 32 = 512
  // sums, two rounds of 256 threads at most.
  for (int idx = threadIdx.x; idx < t.txg * NV * VEC; idx += BN_THREADS) {
    const int tx = idx / (NV * VEC), slot = idx % (NV * VEC);
    float sum = 0.f;
    for (int r = 0; r < t.ty; ++r) sum += red[r * t.txg + tx][slot];
    const int64_t ch = (static_cast<int64_t>(blockIdx.x) * t.txg + tx) * VEC + slot % VEC;
    if (ch < C) atomicAdd(dst[slot / VEC] + ch, static_cast<double>(sum));
  }
}

template <typename T>
__global__ void __launch_bounds__(BN_THREADS, BN_MIN_BLOCKS_REDUCE)
bn_stats_kernel(const T* __restrict__ x, int64_t M, int C, double* __restrict__ sum,
                double* __restrict__ sumsq) {
  const Tile t(C);
  int64_t r0, r1;
  cta_rows(M, &r0, &r1);
  float acc[2][VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[0][i] = acc[1][i] = 0.f;
  const T* base = x + t.group * VEC;
  int64_t r = r0 + t.row;
  for (; r + 3 * t.ty < r1; r += 4 * t.ty) {
    Vec8<T> v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u].raw = ldg16(base + (r + u * t.ty) * C);
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float f = bn_to_float(v[u].e[i]);
        acc[0][i] += f;
        acc[1][i] += f * f;
      }
  }
  for (; r < r1; r += t.ty) {
    Vec8<T> v;
    v.raw = ldg16(base + r * C);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float f = bn_to_float(v.e[i]);
      acc[0][i] += f;
      acc[1][i] += f * f;
    }
  }
  double* const dst[2] = {sum, sumsq};
  reduce_to_global<2>(t, acc, dst, C);
}

// scale/shift of this thread's 8 channels from the fp64 sums.
__device__ __forceinline__ void channel_affine(const double* sum, const double* sumsq,
                                               const float* weight, const float* bias,
                                               int64_t ch0, int64_t M, float eps,
                                               float (&mean)[VEC], float (&invstd)[VEC],
                                               float (&scale)[VEC], float (&shift)[VEC]) {
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const double m = sum[ch0 + i] / static_cast<double>(M);
    double var = sumsq[ch0 + i] / static_cast<double>(M) - m * m;
    if (var < 0.0) var = 0.0;
    const double is = rsqrt(var + static_cast<double>(eps));
    mean[i] = static_cast<float>(m);
    invstd[i] = static_cast<float>(is);
    const float w = weight ? weight[ch0 + i] : 1.f;
    const float b = bias ? bias[ch0 + i] : 0.f;
    scale[i] = w * invstd[i];
    shift[i] = b - mean[i] * scale[i];
  }
}

template <typename T, bool RELU, bool RES>
__global__ void __launch_bounds__(BN_THREADS, BN_MIN_BLOCKS_APPLY)
bn_apply_kernel(const T* __restrict__ x, const T* __restrict__ res, T* __restrict__ y,
                int64_t M, int C, const double* __restrict__ sum,
                const double* __restrict__ sumsq, const float* __restrict__ weight,
                const float* __restrict__ bias, float eps, float momentum,
                float* __restrict__ save_mean, float* __restrict__ save_invstd,
                float* __restrict__ running_mean, float* __restrict__ running_var) {
  const Tile t(C);
  int64_t r0, r1;
  cta_rows(M, &r0, &r1);
  const int64_t ch0 = t.group * VEC;
  float mean[VEC], invstd[VEC], scale[VEC], shift[VEC];
  channel_affine(sum, sumsq, weight, bias, ch0, M, eps, mean, invstd, scale, shift);
  if (blockIdx.y == 0 && t.row == 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      save_mean[ch0 + i] = mean[i];
      save_invstd[ch0 + i] = invstd[i];
      if (running_mean != nullptr) {
        const double m = sum[ch0 + i] / static_cast<double>(M);
        double var = sumsq[ch0 + i] / static_cast<double>(M) - m * m;
        if (var < 0.0) var = 0.0;
        const double unbiased = M > 1 ? var * static_cast<double>(M) / static_cast<double>(M - 1) : var;
        running_mean[ch0 + i] = (1.f - momentum) * running_mean[ch0 + i] + momentum * mean[i];
        running_var[ch0 + i] =
            (1.f - momentum) * running_var[ch0 + i] + momentum * static_cast<float>(unbiased);
      }
    }
  }
  const int64_t off = t.group * VEC;
  auto one = [&](uint4 xv, uint4 rv) {
    Vec8<T> a, b, o;
    a.raw = xv;
    b.raw = rv;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float f = bn_to_float(a.e[i]) * scale[i] + shift[i];
      if (RES) f += bn_to_float(b.e[i]);
      if (RELU) f = fmaxf(f, 0.f);
      o.e[i] = bn_from_float<T>(f);
    }
    return o.raw;
  };
  int64_t r = r0 + t.row;
  for (; r + 3 * t.ty < r1; r += 4 * t.ty) {
    uint4 xv[4], rv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      xv[u] = ldg16(x + (r + u * t.ty) * C + off);
      rv[u] = RES ? ldg16(res + (r + u * t.ty) * C + off) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) stg16(y + (r + u * t.ty) * C + off, one(xv[u], rv[u]));
  }
  for (; r < r1; r += t.ty) {
    const uint4 xv = ldg16(x + r * C + off);
    const uint4 rv = RES ? ldg16(res + r * C + off) : make_uint4(0, 0, 0, 0);
    stg16(y + r * C + off, one(xv, rv));
  }
}

// sum(dz) and sum(dz * xhat) per channel.
template <typename T, bool RELU>
__global__ void __launch_bounds__(BN_THREADS, BN_MIN_BLOCKS_REDUCE)
bn_backward_reduce_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                          const T* __restrict__ x, int64_t M, int C,
                          const float* __restrict__ save_mean,
                          const float* __restrict__ save_invstd, double* __restrict__ sum_dz,
                          double* __restrict__ sum_dz_xhat) {
  const Tile t(C);
  int64_t r0, r1;
  cta_rows(M, &r0, &r1);
  const int64_t off = t.group * VEC;
  float mean[VEC], invstd[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    mean[i] = save_mean[off + i];
    invstd[i] = save_invstd[off + i];
  }
  float acc[2][VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[0][i] = acc[1][i] = 0.f;
  auto one = [&](uint4 dv, uint4 yv, uint4 xv) {
    Vec8<T> d, o, a;
    d.raw = dv;
    o.raw = yv;
    a.raw = xv;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float dz = bn_to_float(d.e[i]);
      if (RELU && !(bn_to_float(o.e[i]) > 0.f)) dz = 0.f;
      acc[0][i] += dz;
      acc[1][i] += dz * (bn_to_float(a.e[i]) - mean[i]) * invstd[i];
    }
  };
  int64_t r = r0 + t.row;
  for (; r + 1 * t.ty < r1; r += 2 * t.ty) {
    uint4 dv[2], yv[2], xv[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t at = (r + u * t.ty) * C + off;
      dv[u] = ldg16(dy + at);
      yv[u] = RELU ? ldg16(y + at) : make_uint4(0, 0, 0, 0);
      xv[u] = ldg16(x + at);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) one(dv[u], yv[u], xv[u]);
  }
  for (; r < r1; r += t.ty) {
    const int64_t at = r * C + off;
    one(ldg16(dy + at), RELU ? ldg16(y + at) : make_uint4(0, 0, 0, 0), ldg16(x + at));
  }
  double* const dst[2] = {sum_dz, sum_dz_xhat};
  reduce_to_global<2>(t, acc, dst, C);
}

template <typename T, bool RELU, bool RES>
__global__ void __launch_bounds__(BN_THREADS, BN_MIN_BLOCKS_APPLY)
bn_backward_apply_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                         const T* __restrict__ x, T* __restrict__ dx, T* __restrict__ dres,
                         int64_t M, int C, const float* __restrict__ weight,
                         const float* __restrict__ save_mean,
                         const float* __restrict__ save_invstd,
                         const double* __restrict__ sum_dz,
                         const double* __restrict__ sum_dz_xhat, float* __restrict__ dweight,
                         float* __restrict__ dbias) {
  const Tile t(C);
  int64_t r0, r1;
  cta_rows(M, &r0, &r1);
  const int64_t off = t.group * VEC;
  float mean[VEC], invstd[VEC], scale[VEC], k1[VEC], k2[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    mean[i] = save_mean[off + i];
    invstd[i] = save_invstd[off + i];
    scale[i] = (weight ? weight[off + i] : 1.f) * invstd[i];
    k1[i] = static_cast<float>(sum_dz[off + i] / static_cast<double>(M));
    k2[i] = static_cast<float>(sum_dz_xhat[off + i] / static_cast<double>(M));
  }
  if (blockIdx.y == 0 && t.row == 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if (dweight) dweight[off + i] = static_cast<float>(sum_dz_xhat[off + i]);
      if (dbias) dbias[off + i] = static_cast<float>(sum_dz[off + i]);
    }
  }
  auto one = [&](uint4 dv, uint4 yv, uint4 xv, uint4* dres_out) {
    Vec8<T> d, o, a, gx, gr;
    d.raw = dv;
    o.raw = yv;
    a.raw = xv;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float dz = bn_to_float(d.e[i]);
      if (RELU && !(bn_to_float(o.e[i]) > 0.f)) dz = 0.f;
      const float xhat = (bn_to_float(a.e[i]) - mean[i]) * invstd[i];
      gx.e[i] = bn_from_float<T>(scale[i] * (dz - k1[i] - xhat * k2[i]));
      gr.e[i] = bn_from_float<T>(dz);
    }
    *dres_out = gr.raw;
    return gx.raw;
  };
  int64_t r = r0 + t.row;
  for (; r + 1 * t.ty < r1; r += 2 * t.ty) {
    uint4 dv[2], yv[2], xv[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t at = (r + u * t.ty) * C + off;
      dv[u] = ldg16(dy + at);
      yv[u] = RELU ? ldg16(y + at) : make_uint4(0, 0, 0, 0);
      xv[u] = ldg16(x + at);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t at = (r + u * t.ty) * C + off;
      uint4 gr;
      stg16(dx + at, one(dv[u], yv[u], xv[u], &gr));
      if (RES) stg16(dres + at, gr);
    }
  }
  for (; r < r1; r += t.ty) {
    const int64_t at = r * C + off;
    uint4 gr;
    stg16(dx + at,
          one(ldg16(dy + at), RELU ? ldg16(y + at) : make_uint4(0, 0, 0, 0), ldg16(x + at), &gr));
    if (RES) stg16(dres + at, gr);
  }
}

dim3 bn_grid(int64_t M, int C) {
  const int cg = C / VEC;
  const int txg = cg < 32 ? cg : 32;
  const int ty = BN_THREADS / txg;
  const int ctiles = cg / txg;
  // About eight CTAs per SM in total, at least 4 * ty rows each.
  int64_t by = (148 * 8 + ctiles - 1) / ctiles;
  const int64_t max_by = (M + 4 * ty - 1) / (4 * ty);
  if (by > max_by) by = max_by;
  if (by < 1) by = 1;
  if (by > 65535) by = 65535;
  return dim3(static_cast<unsigned>(ctiles), static_cast<unsigned>(by), 1);
}

bool bn_shape_ok(int64_t M, int C) {
  if (M < 1 || C < VEC || C % VEC != 0) return false;
  const int cg = C / VEC;
  // Channel groups must tile into CTAs of min(cg, 32) groups, and that width
  // must divide the CTA size.
  const int txg = cg < 32 ? cg : 32;
  return cg % txg == 0 && BN_THREADS % txg == 0;
}

}  // namespace

bool BatchNormSupported(int64_t rows, int channels) { return bn_shape_ok(rows, channels); }

template <typename T>
static cudaError_t ForwardTyped(const void* x, const void* res, void* y, int64_t M, int C,
                                double* sums, const float* weight, const float* bias,
                                float eps, float momentum, float* save_mean,
                                float* save_invstd, float* running_mean, float* running_var,
                                bool relu, cudaStream_t stream) {
  const dim3 grid = bn_grid(M, C);
  double* sum = sums;
  double* sumsq = sums + C;
  bn_stats_kernel<T><<<grid, BN_THREADS, 0, stream>>>(static_cast<const T*>(x), M, C, sum, sumsq);
#define HVD_BN_APPLY(RELU, RES)                                                          \
  bn_apply_kernel<T, RELU, RES><<<grid, BN_THREADS, 0, stream>>>(                         \
      static_cast<const T*>(x), static_cast<const T*>(res), static_cast<T*>(y), M, C, sum, \
      sumsq, weight, bias, eps, momentum, save_mean, save_invstd, running_mean, running_var)
  if (relu && res) HVD_BN_APPLY(true, true);
  else if (relu) HVD_BN_APPLY(true, false);
  else if (res) HVD_BN_APPLY(false, true);
  else HVD_BN_APPLY(false, false);
#undef HVD_BN_APPLY
  return cudaGetLastError();
}

template <typename T>
static cudaError_t BackwardTyped(const void* dy, const void* y, const void* x, void* dx,
                                 void* dres, int64_t M, int C, double* sums,
                                 const float* weight, const float* save_mean,
                                 const float* save_invstd, float* dweight, float* dbias,
                                 bool relu, cudaStream_t stream) {
  const dim3 grid = bn_grid(M, C);
  double* sum_dz = sums;
  double* sum_dz_xhat = sums + C;
  const T* dyt = static_cast<const T*>(dy);
  const T* yt = static_cast<const T*>(y);
  const T* xt = static_cast<const T*>(x);
  if (relu)
    bn_backward_reduce_kernel<T, true><<<grid, BN_THREADS, 0, stream>>>(
        dyt, yt, xt, M, C, save_mean, save_invstd, sum_dz, sum_dz_xhat);
  else
    bn_backward_reduce_kernel<T, false><<<grid, BN_THREADS, 0, stream>>>(
        dyt, yt, xt, M, C, save_mean, save_invstd, sum_dz, sum_dz_xhat);
#define HVD_BN_BWD(RELU, RES)                                                             \
  bn_backward_apply_kernel<T, RELU, RES><<<grid, BN_THREADS, 0, stream>>>(                 \
      dyt, yt, xt, static_cast<T*>(dx), static_cast<T*>(dres), M, C, weight, save_mean,    \
      save_invstd, sum_dz, sum_dz_xhat, dweight, dbias)
  if (relu && dres) HVD_BN_BWD(true, true);
  else if (relu) HVD_BN_BWD(true, false);
  else if (dres) HVD_BN_BWD(false, true);
  else HVD_BN_BWD(false, false);
#undef HVD_BN_BWD
  return cudaGetLastError();
}

cudaError_t LaunchBatchNormForward(const void* x, const void* residual, void* y, int64_t rows,
                                   int channels, bool bf16, double* sums_zeroed,
                                   const float* weight, const float* bias, float eps,
                                   float momentum, float* save_mean, float* save_invstd,
                                   float* running_mean, float* running_var, bool relu,
                                   cudaStream_t stream) {
  if (!bn_shape_ok(rows, channels)) return cudaErrorInvalidValue;
  CountKernelLaunches(2);
  return bf16 ? ForwardTyped<__nv_bfloat16>(x, residual, y, rows, channels, sums_zeroed, weight,
                                            bias, eps, momentum, save_mean, save_invstd,
                                            running_mean, running_var, relu, stream)
              : ForwardTyped<__half>(x, residual, y, rows, channels, sums_zeroed, weight, bias,
                                     eps, momentum, save_mean, save_invstd, running_mean,
                                     running_var, relu, stream);
}

cudaError_t LaunchBatchNormBackward(const void* dy, const void* y, const void* x, void* dx,
                                    void* dresidual, int64_t rows, int channels, bool bf16,
                                    double* sums_zeroed, const float* weight,
                                    const float* save_mean, const float* save_invstd,
                                    float* dweight, float* dbias, bool relu,
                                    cudaStream_t stream) {
  if (!bn_shape_ok(rows, channels)) return cudaErrorInvalidValue;
  CountKernelLaunches(2);
  return bf16 ? BackwardTyped<__nv_bfloat16>(dy, y, x, dx, dresidual, rows, channels,
                                             sums_zeroed, weight, save_mean, save_invstd,
                                             dweight, dbias, relu, stream)
              : BackwardTyped<__half>(dy, y, x, dx, dresidual, rows, channels, sums_zeroed,
                                      weight, save_mean, save_invstd, dweight, dbias, relu,
                                      stream);
}

}  // namespace kern
}  // namespace hvd
