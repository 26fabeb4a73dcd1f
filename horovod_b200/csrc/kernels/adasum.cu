// Adasum across the GPUs of one NVSwitch box, computed on the device over
// peer memory (vector halving, distance doubling).
//
// The fused gradients are packed as fp32 into the local staging buffer. At
// level l (distance d = 2^l) rank r is paired with rank r^d; the pair splits
// the range it still owns in half and each side keeps one half. For that
// half, "a" is the vector held by the lower group and "b" the one held by
// the upper group; one side reads its partner's copy over NVLink. Per tensor,
// dot(a,b), |a|^2 and |b|^2 are accumulated in fp64, published in a scratch
// area, summed over the 2d ranks that jointly hold a and b, and the kept
// half becomes (1 - dot/(2|a|^2)) a + (1 - dot/(2|b|^2)) b. After log2(world)
// levels every rank owns 1/world of the result and reads the other pieces
// from its peers while scattering (postscaled) into the output tensors.
//
// Each phase is its own launch (a grid-wide reduction separates them) and
// starts with a cross-GPU barrier, which also orders it after the peers'
// previous phase.
//
// Device-side counterpart of the host algorithm in
// horovod/common/ops/adasum/adasum.h:194-435, which the reference runs on the
// CPU after copying gradients off the GPU
// (horovod/common/ops/adasum_gpu_operations.cc:197-276).
#include "tensor_walk.cuh"

namespace hvd {
namespace kern {

namespace {

constexpr int THREADS = 512;

struct Range {
  int64_t lo, hi;
};

// Range (in 16-byte vectors) rank r still owns after `levels` halvings.
__device__ __host__ inline Range owned_range(int64_t nvec, int r, int levels) {
  Range g = {0, nvec};
  for (int j = 0; j < levels; ++j) {
    int64_t mid = g.lo + (g.hi - g.lo) / 2;
    if ((r >> j) & 1) g.lo = mid; else g.hi = mid;
  }
  return g;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
adasum_pack_kernel(TensorList tl, SymmCtx ctx, float prescale, double* scratch,
                   int scratch_doubles) {
  constexpr int N = 4;
  const int64_t nvec = tl.offsets[tl.n] / N;
  const int64_t per = (nvec + gridDim.x - 1) / gridDim.x;
  const int64_t lo = blockIdx.x * per, hi = min(lo + per, nvec);
  for (int i = blockIdx.x * THREADS + threadIdx.x; i < scratch_doubles;
       i += gridDim.x * THREADS)
    scratch[i] = 0.0;
  if (lo >= hi) return;
  uint4* stage = reinterpret_cast<uint4*>(ctx.local);
  const bool pre = prescale != 1.0f;
  gather_range<T, float, float, THREADS>(tl, lo, hi, prescale, pre,
                                         [stage](int64_t v, uint4 x) { st16(stage + v, x); });
}

__device__ __forceinline__ void flush_sums(double* dst, int t, double d,
                                           double na, double nb) {
  if (t < 0) return;
  atomicAdd(dst + 3 * t, d);
  atomicAdd(dst + 3 * t + 1, na);
  atomicAdd(dst + 3 * t + 2, nb);
}

__global__ void __launch_bounds__(THREADS)
adasum_dots_kernel(TensorList tl, SymmCtx ctx, int level, uint32_t epoch,
                   double* scratch_level) {
  constexpr int N = 4;
  if (!cta_barrier(ctx, epoch, blockIdx.x, 10 + 2 * level)) return;
  const int64_t nvec = tl.offsets[tl.n] / N;
  const Range keep = owned_range(nvec, ctx.rank, level + 1);
  const int partner = ctx.rank ^ (1 << level);
  const bool lower = ((ctx.rank >> level) & 1) == 0;
  const uint4* mine = reinterpret_cast<const uint4*>(ctx.local);
  const uint4* theirs = reinterpret_cast<const uint4*>(ctx.peers[partner]);
  const uint4* a = lower ? mine : theirs;
  const uint4* bb = lower ? theirs : mine;

  const int64_t len = keep.hi - keep.lo;
  const int64_t per = (len + gridDim.x - 1) / gridDim.x;
  const int64_t lo = keep.lo + blockIdx.x * per, hi = min(lo + per, keep.hi);
  int t = -1;
  double d = 0, na = 0, nb = 0;
  if (lo + threadIdx.x < hi) {
    int cur = find_tensor(tl, (lo + threadIdx.x) * N);
    for (int64_t v = lo + threadIdx.x; v < hi; v += THREADS) {
      const int64_t elem = v * N;
      while (cur + 1 < tl.n && elem >= tl.offsets[cur + 1]) ++cur;
      if (cur != t) {
        flush_sums(scratch_level, t, d, na, nb);
        t = cur;
        d = na = nb = 0;
      }
      WireVec<float> x, y;
      x.raw = ld16(a + v);
      y.raw = ld16(bb + v);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const double xd = x.e[i], yd = y.e[i];
        d += xd * yd;
        na += xd * xd;
        nb += yd * yd;
      }
    }
  }
  // Warp-level pre-reduction when the whole warp ended on the same tensor.
  __syncwarp();
  const int t0 = __shfl_sync(0xffffffffu, t, 0);
  if (__all_sync(0xffffffffu, t == t0)) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      d += __shfl_down_sync(0xffffffffu, d, o);
      na += __shfl_down_sync(0xffffffffu, na, o);
      nb += __shfl_down_sync(0xffffffffu, nb, o);
    }
    if ((threadIdx.x & 31) == 0) flush_sums(scratch_level, t, d, na, nb);
  } else {
    flush_sums(scratch_level, t, d, na, nb);
  }
}

__global__ void __launch_bounds__(THREADS)
adasum_combine_kernel(TensorList tl, SymmCtx ctx, int level, uint32_t epoch,
                      int64_t scratch_level_off) {
  constexpr int N = 4;
  if (!cta_barrier(ctx, epoch, blockIdx.x, 11 + 2 * level)) return;
  const int64_t nvec = tl.offsets[tl.n] / N;
  const Range keep = owned_range(nvec, ctx.rank, level + 1);
  const int partner = ctx.rank ^ (1 << level);
  const bool lower = ((ctx.rank >> level) & 1) == 0;
  uint4* mine = reinterpret_cast<uint4*>(ctx.local);
  const uint4* theirs = reinterpret_cast<const uint4*>(ctx.peers[partner]);
  const int group = 2 << level;
  const int first = ctx.rank / group * group;

  const int64_t len = keep.hi - keep.lo;
  const int64_t per = (len + gridDim.x - 1) / gridDim.x;
  const int64_t lo = keep.lo + blockIdx.x * per, hi = min(lo + per, keep.hi);
  if (lo + threadIdx.x >= hi) return;
  int cur = find_tensor(tl, (lo + threadIdx.x) * N);
  int t = -1;
  float ca = 1.f, cb = 1.f;
  for (int64_t v = lo + threadIdx.x; v < hi; v += THREADS) {
    const int64_t elem = v * N;
    while (cur + 1 < tl.n && elem >= tl.offsets[cur + 1]) ++cur;
    if (cur != t) {
      t = cur;
      double d = 0, na = 0, nb = 0;
      for (int q = 0; q < group; ++q) {
        const volatile double* s = reinterpret_cast<const volatile double*>(
            ctx.peers[first + q] + scratch_level_off);
        d += s[3 * t];
        na += s[3 * t + 1];
        nb += s[3 * t + 2];
      }
      // sqrt(DBL_MIN): below this a squared norm counts as zero.
      const double tiny = 1.4916681462400413e-154;
      ca = static_cast<float>(na >= tiny ? 1.0 - d / (2.0 * na) : 1.0);
      cb = static_cast<float>(nb >= tiny ? 1.0 - d / (2.0 * nb) : 1.0);
    }
    WireVec<float> x, y;
    x.raw = ld16(mine + v);
    y.raw = ld16(theirs + v);
    const float cm = lower ? ca : cb, ct = lower ? cb : ca;
#pragma unroll
    for (int i = 0; i < N; ++i) x.e[i] = cm * x.e[i] + ct * y.e[i];
    st16(mine + v, x.raw);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
adasum_gather_kernel(TensorList tl, SymmCtx ctx, int levels, uint32_t epoch,
                     float postscale) {
  constexpr int N = 4;
  if (!cta_barrier(ctx, epoch, blockIdx.x, 30)) return;
  const int64_t nvec = tl.offsets[tl.n] / N;
  const bool post = postscale != 1.0f;
  for (int q = 0; q < ctx.world; ++q) {
    const Range own = owned_range(nvec, q, levels);
    const int64_t len = own.hi - own.lo;
    const int64_t per = (len + gridDim.x - 1) / gridDim.x;
    const int64_t lo = own.lo + blockIdx.x * per, hi = min(lo + per, own.hi);
    const uint4* src = reinterpret_cast<const uint4*>(ctx.peers[q]);
    scatter_range<T, float, float, THREADS>(tl, lo, hi, postscale, post,
                                            [src](int64_t v) { return ld16(src + v); });
  }
  // Peers may still be reading this rank's piece.
  cta_barrier(ctx, epoch + 1, blockIdx.x, 31);
}

template <typename T>
cudaError_t LaunchTyped(const TensorList& tl, double prescale, double postscale,
                        int64_t scratch_off, int num_ctas, const SymmCtx& ctx,
                        cudaStream_t stream) {
  int levels = 0;
  while ((1 << levels) < ctx.world) ++levels;
  CountKernelLaunches(2 * levels + 2);
  double* scratch = reinterpret_cast<double*>(ctx.local + scratch_off);
  const int per_level = 3 * tl.n;
  adasum_pack_kernel<T><<<num_ctas, THREADS, 0, stream>>>(
      tl, ctx, static_cast<float>(prescale), scratch, per_level * levels);
  uint32_t epoch = ctx.epoch;
  for (int l = 0; l < levels; ++l) {
    adasum_dots_kernel<<<num_ctas, THREADS, 0, stream>>>(
        tl, ctx, l, ++epoch, scratch + static_cast<int64_t>(l) * per_level);
    adasum_combine_kernel<<<num_ctas, THREADS, 0, stream>>>(
        tl, ctx, l, ++epoch,
        scratch_off + static_cast<int64_t>(l) * per_level * sizeof(double));
  }
  ++epoch;
  adasum_gather_kernel<T><<<num_ctas, THREADS, 0, stream>>>(
      tl, ctx, levels, epoch, static_cast<float>(postscale));
  return cudaGetLastError();
}

}  // namespace

cudaError_t LaunchAdasum(const TensorList& tl, DataType dtype, double prescale,
                         double postscale, int64_t scratch_off, int num_ctas,
                         const SymmCtx& ctx, cudaStream_t stream) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  if ((ctx.world & (ctx.world - 1)) != 0) return cudaErrorInvalidValue;
  switch (dtype) {
  case DataType::FLOAT32:
    return LaunchTyped<float>(tl, prescale, postscale, scratch_off, num_ctas, ctx, stream);
  case DataType::FLOAT16:
    return LaunchTyped<__half>(tl, prescale, postscale, scratch_off, num_ctas, ctx, stream);
  case DataType::BFLOAT16:
    return LaunchTyped<__nv_bfloat16>(tl, prescale, postscale, scratch_off, num_ctas, ctx, stream);
  default:
    return cudaErrorInvalidValue;
  }
}

}  // namespace kern
}  // namespace hvd
