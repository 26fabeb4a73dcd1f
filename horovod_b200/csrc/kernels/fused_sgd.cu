// Multi-tensor SGD (momentum, weight decay, Nesterov) in one launch over a
// list of fp32 tensors: every parameter, gradient and momentum element is
// read once and written once, instead of the four to five elementwise passes
// (or, for tensors whose layout defeats the foreach fast path, one launch per
// tensor per pass) of the framework's optimizer.
//
// The reference has no counterpart (the optimizer is the framework's,
// horovod/torch/optimizer.py:249-325 only wraps its step()).
#include "kernels.h"

namespace hvd {
namespace kern {

namespace {

constexpr int SGD_THREADS = 256;

__global__ void __launch_bounds__(SGD_THREADS)
fused_sgd_kernel(SgdTensors t, float lr, float momentum, float dampening, float weight_decay,
                 bool nesterov, bool first_step, bool maximize) {
  for (int c = blockIdx.x; c < t.n_chunks; c += gridDim.x) {
    const int ti = t.chunk_tensor[c];
    const int64_t start = t.chunk_start[c];
    const int64_t n = min(t.chunk_elems, t.counts[ti] - start);
    float* p = t.params[ti] + start;
    const float* g = t.grads[ti] + start;
    float* b = (t.bufs != nullptr && t.bufs[ti] != nullptr) ? t.bufs[ti] + start : nullptr;
    auto update = [&](float pv, float gv, float bv, float* b_out) {
      if (maximize) gv = -gv;
      if (weight_decay != 0.f) gv = fmaf(weight_decay, pv, gv);
      if (momentum != 0.f) {
        bv = first_step ? gv : fmaf(momentum, bv, (1.f - dampening) * gv);
        *b_out = bv;
        gv = nesterov ? fmaf(momentum, bv, gv) : bv;
      }
      return fmaf(-lr, gv, pv);
    };
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       reinterpret_cast<uintptr_t>(b)) & 15) == 0;
    int64_t done = 0;
    if (vec) {
      const int64_t nv = n >> 2;
      float4* p4 = reinterpret_cast<float4*>(p);
      const float4* g4 = reinterpret_cast<const float4*>(g);
      float4* b4 = reinterpret_cast<float4*>(b);
      for (int64_t i = threadIdx.x; i < nv; i += SGD_THREADS) {
        float4 pv = p4[i];
        const float4 gv = __ldcs(g4 + i);
        float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b != nullptr && !first_step) bv = b4[i];
        float4 bo = bv;
        pv.x = update(pv.x, gv.x, bv.x, &bo.x);
        pv.y = update(pv.y, gv.y, bv.y, &bo.y);
        pv.z = update(pv.z, gv.z, bv.z, &bo.z);
        pv.w = update(pv.w, gv.w, bv.w, &bo.w);
        p4[i] = pv;
        if (b != nullptr && momentum != 0.f) b4[i] = bo;
      }
      done = nv << 2;
    }
    for (int64_t i = done + threadIdx.x; i < n; i += SGD_THREADS) {
      float bo = 0.f;
      const float bv = (b != nullptr && !first_step) ? b[i] : 0.f;
      p[i] = update(p[i], g[i], bv, &bo);
      if (b != nullptr && momentum != 0.f) b[i] = bo;
    }
  }
}

}  // namespace

cudaError_t LaunchFusedSgd(const SgdTensors& t, float lr, float momentum, float dampening,
                           float weight_decay, bool nesterov, bool first_step, bool maximize,
                           cudaStream_t stream) {
  if (t.n_chunks <= 0) return cudaSuccess;
  if (t.chunk_elems <= 0 || (t.chunk_elems & 3) != 0) return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  const int grid = t.n_chunks < 148 * 8 ? t.n_chunks : 148 * 8;
  fused_sgd_kernel<<<grid, SGD_THREADS, 0, stream>>>(t, lr, momentum, dampening, weight_decay,
                                                     nesterov, first_step, maximize);
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace hvd
