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

// Adds one CTA's partial sums for tensor t to the level's scratch record.
__device__ __forceinline__ void block_flush_sums(double* dst, int t, double d, double na,
                                                 double nb) {
  __shared__ double part[THREADS / 32][3];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    d += __shfl_down_sync(0xffffffffu, d, o);
    na += __shfl_down_sync(0xffffffffu, na, o);
    nb += __shfl_down_sync(0xffffffffu, nb, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    part[warp][0] = d;
    part[warp][1] = na;
    part[warp][2] = nb;
  }
  __syncthreads();
  if (threadIdx.x < 3) {
    double sum = 0;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) sum += part[w][threadIdx.x];
    if (sum != 0.0) atomicAdd(dst + 3 * t + threadIdx.x, sum);
  }
  __syncthreads();  // `part` is reused for the next tensor
}

__device__ __forceinline__ void accumulate(uint4 xa, uint4 xb, double& d, double& na,
                                           double& nb) {
  WireVec<float> x, y;
  x.raw = xa;
  y.raw = xb;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const double xd = x.e[i], yd = y.e[i];
    d += xd * yd;
    na += xd * xd;
    nb += yd * yd;
  }
}

// Per tensor: dot(a,b), |a|^2, |b|^2 over this CTA's slice of the kept half,
// tensor by tensor (tight, four-way unrolled inner loop; the padding between
// tensors holds zeros and adds nothing).
__global__ void __launch_bounds__(THREADS)
adasum_dots_kernel(TensorList tl, SymmCtx ctx, int level, uint32_t epoch,
                   double* scratch_level, int64_t copy_off) {
  constexpr int N = 4;
  if (!cta_barrier(ctx, epoch, blockIdx.x, 10 + 2 * level)) return;
  const int64_t nvec = tl.offsets[tl.n] / N;
  const Range keep = owned_range(nvec, ctx.rank, level + 1);
  const int partner = ctx.rank ^ (1 << level);
  const bool lower = ((ctx.rank >> level) & 1) == 0;
  const uint4* mine = reinterpret_cast<const uint4*>(ctx.local);
  const uint4* theirs = reinterpret_cast<const uint4*>(ctx.peers[partner]);
  // The partner's half crosses NVLink once: while it is read for the dot
  // products it is also written to a local copy (vector v of the kept range
  // at copy[v - keep.lo]) that the combine kernel reads instead.
  uint4* copy = copy_off >= 0 ? reinterpret_cast<uint4*>(ctx.local + copy_off) - keep.lo : nullptr;

  const int64_t len = keep.hi - keep.lo;
  const int64_t per = (len + gridDim.x - 1) / gridDim.x;
  const int64_t lo = keep.lo + blockIdx.x * per, hi = min(lo + per, keep.hi);
  if (lo >= hi) return;  // whole CTA
  for (int t = find_tensor(tl, lo * N); t < tl.n; ++t) {
    const int64_t toff = tl.offsets[t];
    if (toff >= hi * N) break;
    const int64_t v0 = max(lo, toff / N), v1 = min(hi, tl.offsets[t + 1] / N);
    double d = 0, na = 0, nb = 0;
    int64_t v = v0 + threadIdx.x;
    for (; v + 3 * THREADS < v1; v += 4 * THREADS) {
      uint4 xm[4], xt[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        xm[u] = ld16(mine + v + u * THREADS);
        xt[u] = ld16(theirs + v + u * THREADS);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (copy != nullptr) st16(copy + v + u * THREADS, xt[u]);
        if (lower)
          accumulate(xm[u], xt[u], d, na, nb);
        else
          accumulate(xt[u], xm[u], d, na, nb);
      }
    }
    for (; v < v1; v += THREADS) {
      const uint4 xm = ld16(mine + v), xt = ld16(theirs + v);
      if (copy != nullptr) st16(copy + v, xt);
      if (lower)
        accumulate(xm, xt, d, na, nb);
      else
        accumulate(xt, xm, d, na, nb);
    }
    block_flush_sums(scratch_level, t, d, na, nb);
  }
}

// kept half <- ca * a + cb * b with the per-tensor coefficients computed from
// the sums of all ranks that jointly hold a and b.
__global__ void __launch_bounds__(THREADS)
adasum_combine_kernel(TensorList tl, SymmCtx ctx, int level, uint32_t epoch,
                      int64_t scratch_level_off, int64_t copy_off) {
  constexpr int N = 4;
  if (!cta_barrier(ctx, epoch, blockIdx.x, 11 + 2 * level)) return;
  const int64_t nvec = tl.offsets[tl.n] / N;
  const Range keep = owned_range(nvec, ctx.rank, level + 1);
  const int partner = ctx.rank ^ (1 << level);
  const bool lower = ((ctx.rank >> level) & 1) == 0;
  uint4* mine = reinterpret_cast<uint4*>(ctx.local);
  // The partner's half: the local copy the dots kernel made, if there is one.
  const uint4* theirs =
      copy_off >= 0 ? reinterpret_cast<const uint4*>(ctx.local + copy_off) - keep.lo
                    : reinterpret_cast<const uint4*>(ctx.peers[partner]);
  const int group = 2 << level;
  const int first = ctx.rank / group * group;
  __shared__ float coeff[2];
  __shared__ double s_sums[3 * SYMM_MAX_RANKS];

  const int64_t len = keep.hi - keep.lo;
  const int64_t per = (len + gridDim.x - 1) / gridDim.x;
  const int64_t lo = keep.lo + blockIdx.x * per, hi = min(lo + per, keep.hi);
  if (lo >= hi) return;  // whole CTA
  for (int t = find_tensor(tl, lo * N); t < tl.n; ++t) {
    const int64_t toff = tl.offsets[t];
    if (toff >= hi * N) break;
    const int64_t v0 = max(lo, toff / N), v1 = min(hi, tl.offsets[t + 1] / N);
    // The three sums of every rank of the group, one peer read per thread
    // (all in flight together), then summed in rank order.
    if (threadIdx.x < 3 * group) {
      const int q = threadIdx.x / 3, c = threadIdx.x % 3;
      const volatile double* s = reinterpret_cast<const volatile double*>(
          ctx.peers[first + q] + scratch_level_off);
      s_sums[threadIdx.x] = s[3 * t + c];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double d = 0, na = 0, nb = 0;
      for (int q = 0; q < group; ++q) {
        d += s_sums[3 * q];
        na += s_sums[3 * q + 1];
        nb += s_sums[3 * q + 2];
      }
      // sqrt(DBL_MIN): below this a squared norm counts as zero.
      const double tiny = 1.4916681462400413e-154;
      coeff[0] = static_cast<float>(na >= tiny ? 1.0 - d / (2.0 * na) : 1.0);
      coeff[1] = static_cast<float>(nb >= tiny ? 1.0 - d / (2.0 * nb) : 1.0);
    }
    __syncthreads();
    const float cm = lower ? coeff[0] : coeff[1], ct = lower ? coeff[1] : coeff[0];
    auto mix = [&](uint4 xm, uint4 xt) {
      WireVec<float> x, y;
      x.raw = xm;
      y.raw = xt;
#pragma unroll
      for (int i = 0; i < N; ++i) x.e[i] = cm * x.e[i] + ct * y.e[i];
      return x.raw;
    };
    int64_t v = v0 + threadIdx.x;
    for (; v + 3 * THREADS < v1; v += 4 * THREADS) {
      uint4 xm[4], xt[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        xm[u] = ld16(mine + v + u * THREADS);
        xt[u] = ld16(theirs + v + u * THREADS);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) st16(mine + v + u * THREADS, mix(xm[u], xt[u]));
    }
    for (; v < v1; v += THREADS) st16(mine + v, mix(ld16(mine + v), ld16(theirs + v)));
    __syncthreads();  // `coeff` is rewritten for the next tensor
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
                        int64_t scratch_off, int64_t copy_off, int num_ctas,
                        const SymmCtx& ctx, cudaStream_t stream) {
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
        tl, ctx, l, ++epoch, scratch + static_cast<int64_t>(l) * per_level, copy_off);
    adasum_combine_kernel<<<num_ctas, THREADS, 0, stream>>>(
        tl, ctx, l, ++epoch,
        scratch_off + static_cast<int64_t>(l) * per_level * sizeof(double), copy_off);
  }
  ++epoch;
  adasum_gather_kernel<T><<<num_ctas, THREADS, 0, stream>>>(
      tl, ctx, levels, epoch, static_cast<float>(postscale));
  return cudaGetLastError();
}

}  // namespace

cudaError_t LaunchAdasum(const TensorList& tl, DataType dtype, double prescale,
                         double postscale, int64_t scratch_off, int num_ctas,
                         const SymmCtx& ctx, cudaStream_t stream, int64_t copy_off) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  if ((ctx.world & (ctx.world - 1)) != 0) return cudaErrorInvalidValue;
  switch (dtype) {
  case DataType::FLOAT32:
    return LaunchTyped<float>(tl, prescale, postscale, scratch_off, copy_off, num_ctas, ctx, stream);
  case DataType::FLOAT16:
    return LaunchTyped<__half>(tl, prescale, postscale, scratch_off, copy_off, num_ctas, ctx, stream);
  case DataType::BFLOAT16:
    return LaunchTyped<__nv_bfloat16>(tl, prescale, postscale, scratch_off, copy_off, num_ctas, ctx, stream);
  default:
    return cudaErrorInvalidValue;
  }
}

}  // namespace kern
}  // namespace hvd
