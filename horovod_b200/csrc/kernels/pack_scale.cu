// Stand-alone batched pack/unpack and scale kernels for the NCCL path (where
// the collective itself is a library call on a contiguous fusion buffer) and
// for odd cases the fused kernels do not cover.
//
// Same job as the reference's batched_memcpy_k / batched_scaled_memcpy_k /
// scale_buffer_k (horovod/common/ops/cuda/cuda_kernels.cu:44-321), with the
// tensor list in device memory instead of a 160-entry by-value struct, so one
// launch handles any number of tensors, and with an optional cast between
// the tensor type and a 16-bit wire type.
#include <atomic>

#include "tensor_walk.cuh"

namespace hvd {
namespace kern {

namespace {

constexpr int THREADS = 512;

template <typename T, typename W, bool TO_BUFFER>
__global__ void __launch_bounds__(THREADS)
pack_unpack_kernel(TensorList tl, uint4* buffer, typename ScaleT<T>::type scale) {
  using S = typename ScaleT<T>::type;
  constexpr int N = 16 / sizeof(W);
  const int64_t nvec = tl.offsets[tl.n] / N;
  const int64_t per = (nvec + gridDim.x - 1) / gridDim.x;
  const int64_t lo = blockIdx.x * per, hi = min(lo + per, nvec);
  if (lo >= hi) return;
  const bool do_scale = scale != S(1);
  if constexpr (TO_BUFFER)
    gather_range<T, W, S, THREADS>(tl, lo, hi, scale, do_scale,
                                   [buffer](int64_t v, uint4 x) { st16(buffer + v, x); });
  else
    scatter_range<T, W, S, THREADS>(tl, lo, hi, scale, do_scale,
                                    [buffer](int64_t v) { return ld16(buffer + v); });
}

template <typename T, typename W>
cudaError_t LaunchPU(const TensorList& tl, void* buffer, double scale,
                     bool to_buffer, int64_t approx_vecs, cudaStream_t stream) {
  using S = typename ScaleT<T>::type;
  int ctas = static_cast<int>(
      std::min<int64_t>(592, std::max<int64_t>(1, approx_vecs / (THREADS * 4))));
  if (to_buffer)
    pack_unpack_kernel<T, W, true><<<ctas, THREADS, 0, stream>>>(
        tl, static_cast<uint4*>(buffer), static_cast<S>(scale));
  else
    pack_unpack_kernel<T, W, false><<<ctas, THREADS, 0, stream>>>(
        tl, static_cast<uint4*>(buffer), static_cast<S>(scale));
  return cudaGetLastError();
}

template <typename T>
__global__ void scale_kernel(const T* in, T* out, int64_t n,
                             typename ScaleT<T>::type scale) {
  using S = typename ScaleT<T>::type;
  constexpr int N = 16 / sizeof(T);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(in) |
                         reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  int64_t done = 0;
  if (aligned) {
    const int64_t nvec = n / N;
    for (int64_t v = tid; v < nvec; v += stride) {
      WireVec<T> w;
      w.raw = ld16_stream(reinterpret_cast<const uint4*>(in) + v);
#pragma unroll
      for (int i = 0; i < N; ++i) w.e[i] = scale_cast<T, T, S>(w.e[i], scale, true);
      st16_stream(reinterpret_cast<uint4*>(out) + v, w.raw);
    }
    done = nvec * N;
  }
  for (int64_t i = done + tid; i < n; i += stride)
    out[i] = scale_cast<T, T, S>(in[i], scale, true);
}

}  // namespace

namespace {
std::atomic<uint64_t> g_launches{0};
}
uint64_t KernelLaunchCount() { return g_launches.load(); }
void CountKernelLaunches(int n) { g_launches.fetch_add(static_cast<uint64_t>(n)); }

cudaError_t LaunchPackUnpack(const TensorList& tl, DataType dtype, DataType wire,
                             void* buffer, double scale, bool to_buffer,
                             int64_t total_elements, cudaStream_t stream) {
  const int64_t approx =
      total_elements * static_cast<int64_t>(DataTypeSize(wire)) / 16;
  CountKernelLaunches(1);
#define HVD_PU(T, W) return LaunchPU<T, W>(tl, buffer, scale, to_buffer, approx, stream)
  if (dtype == DataType::FLOAT32 && wire == DataType::BFLOAT16) HVD_PU(float, __nv_bfloat16);
  if (dtype == DataType::FLOAT32 && wire == DataType::FLOAT16) HVD_PU(float, __half);
  if (dtype != wire) return cudaErrorInvalidValue;
  switch (dtype) {
  case DataType::FLOAT32: HVD_PU(float, float);
  case DataType::FLOAT16: HVD_PU(__half, __half);
  case DataType::BFLOAT16: HVD_PU(__nv_bfloat16, __nv_bfloat16);
  case DataType::FLOAT64: HVD_PU(double, double);
  case DataType::INT32: HVD_PU(int32_t, int32_t);
  case DataType::INT64: HVD_PU(int64_t, int64_t);
  case DataType::UINT8:
  case DataType::BOOL: HVD_PU(uint8_t, uint8_t);
  case DataType::INT8: HVD_PU(int8_t, int8_t);
  case DataType::INT16: HVD_PU(int16_t, int16_t);
  case DataType::UINT16: HVD_PU(uint16_t, uint16_t);
  default: return cudaErrorInvalidValue;
  }
#undef HVD_PU
}

cudaError_t LaunchScaleBuffer(const void* in, void* out, int64_t count,
                              DataType dtype, double scale, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  CountKernelLaunches(1);
  const int threads = 256;
  const int blocks = static_cast<int>(
      std::min<int64_t>(1184, (count + threads * 8 - 1) / (threads * 8)));
#define HVD_SC(T)                                                             \
  scale_kernel<T><<<blocks, threads, 0, stream>>>(                            \
      static_cast<const T*>(in), static_cast<T*>(out), count,                 \
      static_cast<typename ScaleT<T>::type>(scale));                          \
  return cudaGetLastError()
  switch (dtype) {
  case DataType::FLOAT32: HVD_SC(float);
  case DataType::FLOAT16: HVD_SC(__half);
  case DataType::BFLOAT16: HVD_SC(__nv_bfloat16);
  case DataType::FLOAT64: HVD_SC(double);
  case DataType::INT32: HVD_SC(int32_t);
  case DataType::INT64: HVD_SC(int64_t);
  case DataType::UINT8: HVD_SC(uint8_t);
  case DataType::INT8: HVD_SC(int8_t);
  case DataType::INT16: HVD_SC(int16_t);
  case DataType::UINT16: HVD_SC(uint16_t);
  default: return cudaErrorInvalidValue;
  }
#undef HVD_SC
}

}  // namespace kern
}  // namespace hvd
