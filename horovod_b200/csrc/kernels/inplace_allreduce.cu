// In-place allreduce on tensors that already live in symmetric memory (the
// "symmetric heap"): no staging, no pack, no unpack. Every rank holds the
// tensor at the same offset of its arena, so rank r sums chunk r straight out
// of all ranks' tensors (multimem.ld_reduce through the NVSwitch, or peer
// loads) and writes the scaled result straight back into all of them
// (multimem.st, or peer stores). Local HBM traffic is only what NVLink
// delivers; the whole op is one launch with two cross-GPU barriers.
//
// A launch covers a list of byte ranges (the gradients of one fused
// response, adjacent ones merged). Ranges start on 16-byte boundaries; a
// ragged tail shorter than 16 bytes is reduced element by element over peer
// pointers.
//
// The reference has no counterpart: its allreduce always stages through a
// fusion buffer around ncclAllReduce
// (horovod/common/ops/nccl_operations.cc:156-214).
#include "tensor_walk.cuh"

namespace hvd {
namespace kern {

namespace {

constexpr int THREADS = 512;

template <typename W>
__device__ __forceinline__ uint4 scale_vec(uint4 raw, float scale, bool do_scale) {
  if (!do_scale) return raw;
  constexpr int N = 16 / sizeof(W);
  WireVec<W> v;
  v.raw = raw;
#pragma unroll
  for (int i = 0; i < N; ++i) v.e[i] = scale_cast<W>(v.e[i], scale, true);
  return v.raw;
}
template <>
__device__ __forceinline__ uint4 scale_vec<double>(uint4 raw, float scale, bool do_scale) {
  if (!do_scale) return raw;
  WireVec<double> v;
  v.raw = raw;
  v.e[0] *= static_cast<double>(scale);
  v.e[1] *= static_cast<double>(scale);
  return v.raw;
}

template <typename W, bool NVLS, int WORLD>
__device__ __forceinline__ void reduce_vectors(const SymmCtx& ctx, int64_t byte_off,
                                               int64_t v_lo, int64_t v_hi,
                                               float scale, bool do_scale) {
  // v_lo/v_hi index 16-byte vectors relative to byte_off.
  if constexpr (NVLS) {
    uint4* mc = reinterpret_cast<uint4*>(ctx.mc + byte_off);
    int64_t v = v_lo + threadIdx.x;
    for (; v + 3 * THREADS < v_hi; v += 4 * THREADS) {
      uint4 x0 = Multimem<W>::ld_reduce(mc + v);
      uint4 x1 = Multimem<W>::ld_reduce(mc + v + THREADS);
      uint4 x2 = Multimem<W>::ld_reduce(mc + v + 2 * THREADS);
      uint4 x3 = Multimem<W>::ld_reduce(mc + v + 3 * THREADS);
      multimem_st16(mc + v, scale_vec<W>(x0, scale, do_scale));
      multimem_st16(mc + v + THREADS, scale_vec<W>(x1, scale, do_scale));
      multimem_st16(mc + v + 2 * THREADS, scale_vec<W>(x2, scale, do_scale));
      multimem_st16(mc + v + 3 * THREADS, scale_vec<W>(x3, scale, do_scale));
    }
    for (; v < v_hi; v += THREADS)
      multimem_st16(mc + v, scale_vec<W>(Multimem<W>::ld_reduce(mc + v), scale, do_scale));
  } else {
    constexpr int UNROLL = WORLD <= 2 ? 4 : (WORLD <= 4 ? 2 : 1);
    const uint4* src[WORLD];
    uint4* dst[WORLD];
#pragma unroll
    for (int i = 0; i < WORLD; ++i) {
      int p = ctx.rank + i;
      if (p >= WORLD) p -= WORLD;
      src[i] = reinterpret_cast<const uint4*>(ctx.peers[p] + byte_off);
      dst[i] = reinterpret_cast<uint4*>(ctx.peers[p] + byte_off);
    }
    int64_t v = v_lo + threadIdx.x;
    for (; v + (UNROLL - 1) * THREADS < v_hi; v += UNROLL * THREADS) {
      uint4 in[UNROLL][WORLD];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int i = 0; i < WORLD; ++i) in[u][i] = ld16(src[i] + v + u * THREADS);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        VecAcc<W> acc;
        acc.zero();
#pragma unroll
        for (int i = 0; i < WORLD; ++i) acc.add(in[u][i]);
        const uint4 sum = scale_vec<W>(acc.pack(), scale, do_scale);
#pragma unroll
        for (int i = 0; i < WORLD; ++i) st16(dst[i] + v + u * THREADS, sum);
      }
    }
    for (; v < v_hi; v += THREADS) {
      VecAcc<W> acc;
      acc.zero();
#pragma unroll
      for (int i = 0; i < WORLD; ++i) acc.add(ld16(src[i] + v));
      const uint4 sum = scale_vec<W>(acc.pack(), scale, do_scale);
#pragma unroll
      for (int i = 0; i < WORLD; ++i) st16(dst[i] + v, sum);
    }
  }
}

// Elements of a ragged tail (fewer than 16 bytes), over peer pointers.
template <typename W>
__device__ __forceinline__ void reduce_tail(const SymmCtx& ctx, int64_t byte_off,
                                            int n_elems, float scale, bool do_scale) {
  using A = typename Acc<W>::type;
  if (threadIdx.x >= n_elems) return;
  A acc = A(0);
  for (int p = 0; p < ctx.world; ++p) {
    const volatile W* s = reinterpret_cast<const volatile W*>(ctx.peers[p] + byte_off);
    W x;
    // volatile element read (never cached in L1)
    const volatile unsigned char* b =
        reinterpret_cast<const volatile unsigned char*>(s + threadIdx.x);
    unsigned char* xb = reinterpret_cast<unsigned char*>(&x);
    for (int k = 0; k < static_cast<int>(sizeof(W)); ++k) xb[k] = b[k];
    acc += to_acc<A, W>(x);
  }
  W out = from_acc<W, A>(acc);
  if (do_scale) {
    if constexpr (std::is_same<W, double>::value) out *= static_cast<double>(scale);
    else out = scale_cast<W>(out, scale, true);
  }
  for (int p = 0; p < ctx.world; ++p) {
    volatile unsigned char* d =
        reinterpret_cast<volatile unsigned char*>(ctx.peers[p] + byte_off) +
        threadIdx.x * sizeof(W);
    const unsigned char* ob = reinterpret_cast<const unsigned char*>(&out);
    for (int k = 0; k < static_cast<int>(sizeof(W)); ++k) d[k] = ob[k];
  }
}

// Vectors [lo, hi) of the fused vector space, which may span several ranges.
template <typename W, bool NVLS, int WORLD>
__device__ __forceinline__ void reduce_span(const RangeList& rl, const SymmCtx& ctx,
                                            int64_t lo, int64_t hi, float scale,
                                            bool do_scale) {
  if (lo >= hi) return;
  // first range that may contain `lo`
  int t = 0;
  {
    int a = 0, z = rl.n - 1;
    while (a < z) {
      int mid = (a + z + 1) >> 1;
      if (rl.vec_start[mid] <= lo) a = mid; else z = mid - 1;
    }
    t = a;
  }
  for (; t < rl.n; ++t) {
    const int64_t r0 = rl.vec_start[t];
    if (r0 >= hi) break;
    const int64_t r1 = rl.vec_start[t + 1];
    const int64_t full = rl.bytes[t] >> 4;  // whole vectors in this range
    const int64_t v0 = max(lo, r0) - r0, v1 = min(hi, r1) - r0;
    reduce_vectors<W, NVLS, WORLD>(ctx, rl.byte_off[t], v0, min(v1, full), scale, do_scale);
    if (v1 > full && full >= v0) {
      // this span owns the ragged last vector of the range
      const int tail = static_cast<int>((rl.bytes[t] & 15) / sizeof(W));
      reduce_tail<W>(ctx, rl.byte_off[t] + (full << 4), tail, scale, do_scale);
    }
  }
}

// INLINE: the range list rides in the kernel parameters and is copied to
// shared memory first (parameter reads with compile-time offsets only); else
// it is read from device memory.
template <typename W, bool NVLS, int WORLD, bool INLINE>
__global__ void __launch_bounds__(THREADS)
inplace_allreduce_kernel(const InlineRanges inl, const RangeList list_dev,
                         SymmCtx ctx, float scale, TileSchedule sched) {
  __shared__ int64_t s_vec_start[INLINE ? INLINE_TENSORS + 1 : 1];
  __shared__ int64_t s_byte_off[INLINE ? INLINE_TENSORS : 1];
  __shared__ int64_t s_bytes[INLINE ? INLINE_TENSORS : 1];
  RangeList rl = list_dev;
  if constexpr (INLINE) {
#pragma unroll
    for (int i = 0; i < INLINE_TENSORS; ++i) {
      if (threadIdx.x == i && i < inl.n) {
        s_vec_start[i] = inl.vec_start[i];
        s_byte_off[i] = inl.byte_off[i];
        s_bytes[i] = inl.bytes[i];
      }
    }
#pragma unroll
    for (int i = 1; i <= INLINE_TENSORS; ++i)
      if (threadIdx.x == 32 && i == inl.n) s_vec_start[i] = inl.vec_start[i];
    __syncthreads();
    rl.n = inl.n;
    rl.vec_start = s_vec_start;
    rl.byte_off = s_byte_off;
    rl.bytes = s_bytes;
  }
  const int b = blockIdx.x, G = gridDim.x;
  const bool do_scale = scale != 1.0f;
  // Everybody's producers have finished once their kernel is here.
  trace_mark(ctx, 0);
  const uint32_t token =
      symm_token(ctx.epoch, rl.byte_off[0], rl.vec_start[rl.n] << 4, rl.n);
  if (!cta_barrier_token(ctx, ctx.epoch + 1, b, 1, token)) return;
  trace_mark(ctx, 2);

  const int64_t total = rl.vec_start[rl.n];  // vectors, ragged tails count as one
  const int64_t per_rank = (total + ctx.world - 1) / ctx.world;
  const int64_t mine_lo = ctx.rank * per_rank;
  const int64_t mine_hi = min(mine_lo + per_rank, total);
  if (sched.counter == nullptr) {
    // Static split: CTA b owns slice b of this rank's chunk.
    const int64_t per_cta = (per_rank + G - 1) / G;
    const int64_t lo = mine_lo + b * per_cta;
    reduce_span<W, NVLS, WORLD>(rl, ctx, lo, min(lo + per_cta, mine_hi), scale, do_scale);
  } else {
    // Dynamic split for large messages: CTAs draw tiles from a counter, so
    // SMs that get less NVLink or HBM bandwidth simply take fewer tiles and
    // nobody waits for a straggler. The counter only ever grows: this launch
    // owns the values [base, base + ntiles + gridDim.x).
    __shared__ unsigned long long s_tile;
    const int64_t ntiles = (mine_hi - mine_lo + sched.tile_vecs - 1) / sched.tile_vecs;
    for (;;) {
      if (threadIdx.x == 0) s_tile = atomicAdd(sched.counter, 1ULL) - sched.base;
      __syncthreads();
      const int64_t t = static_cast<int64_t>(s_tile);
      __syncthreads();
      if (t < 0 || t >= ntiles) break;  // t < 0: counter behind the host (failed launch)
      const int64_t lo = mine_lo + t * sched.tile_vecs;
      reduce_span<W, NVLS, WORLD>(rl, ctx, lo, min(lo + sched.tile_vecs, mine_hi), scale,
                                  do_scale);
    }
  }
  // Results are in every rank's tensor before anyone's kernel completes.
  trace_mark(ctx, 3);
  cta_barrier(ctx, ctx.epoch + 2, b, 2);
  trace_mark(ctx, 4);
}

template <typename W, bool NVLS>
cudaError_t LaunchWorld(const InlineRanges& inl, const RangeList& rl, int num_ctas,
                        const SymmCtx& ctx, float scale, cudaStream_t stream,
                        const TileSchedule& sched) {
#define HVD_IP(WD)                                                                      \
  do {                                                                                  \
    if (inl.n > 0)                                                                      \
      inplace_allreduce_kernel<W, NVLS, WD, true><<<num_ctas, THREADS, 0, stream>>>(    \
          inl, rl, ctx, scale, sched);                                                  \
    else                                                                                \
      inplace_allreduce_kernel<W, NVLS, WD, false><<<num_ctas, THREADS, 0, stream>>>(   \
          inl, rl, ctx, scale, sched);                                                  \
  } while (0)
  if constexpr (NVLS) {
    HVD_IP(8);  // WORLD is unused on the multimem path
  } else {
    switch (ctx.world) {
    case 2: HVD_IP(2); break;
    case 3: HVD_IP(3); break;
    case 4: HVD_IP(4); break;
    case 5: HVD_IP(5); break;
    case 6: HVD_IP(6); break;
    case 7: HVD_IP(7); break;
    case 8: HVD_IP(8); break;
    default: return cudaErrorInvalidValue;
    }
  }
#undef HVD_IP
  return cudaGetLastError();
}

}  // namespace

cudaError_t LaunchInplaceAllreduce(const RangeList& ranges, DataType dtype,
                                   double scale, bool use_nvls, int num_ctas,
                                   const SymmCtx& ctx, cudaStream_t stream,
                                   const InlineRanges* inline_ranges,
                                   const TileSchedule* schedule) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  if (ctx.world < 2) return cudaErrorInvalidValue;
  static const InlineRanges kNoInline = {};
  const InlineRanges& inl = inline_ranges ? *inline_ranges : kNoInline;
  const float s = static_cast<float>(scale);
  const bool nvls = use_nvls && ctx.mc != nullptr;
  static const TileSchedule kStatic = {nullptr, 0, 0};
  const TileSchedule& sched = schedule ? *schedule : kStatic;
  CountKernelLaunches(1);
  switch (dtype) {
  case DataType::FLOAT32:
    return nvls ? LaunchWorld<float, true>(inl, ranges, num_ctas, ctx, s, stream, sched)
                : LaunchWorld<float, false>(inl, ranges, num_ctas, ctx, s, stream, sched);
  case DataType::FLOAT16:
    return nvls ? LaunchWorld<__half, true>(inl, ranges, num_ctas, ctx, s, stream, sched)
                : LaunchWorld<__half, false>(inl, ranges, num_ctas, ctx, s, stream, sched);
  case DataType::BFLOAT16:
    return nvls ? LaunchWorld<__nv_bfloat16, true>(inl, ranges, num_ctas, ctx, s, stream, sched)
                : LaunchWorld<__nv_bfloat16, false>(inl, ranges, num_ctas, ctx, s, stream, sched);
  case DataType::FLOAT64:
    return LaunchWorld<double, false>(inl, ranges, num_ctas, ctx, s, stream, sched);
  default:
    return cudaErrorInvalidValue;
  }
}

}  // namespace kern
}  // namespace hvd
