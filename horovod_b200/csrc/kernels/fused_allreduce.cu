// Fused multi-tensor allreduce over NVLink: one launch gathers the tensors
// (prescale + cast to the wire type), reduces across GPUs and scatters the
// result back (cast + postscale). Three cross-GPU algorithms share the
// gather/scatter code:
//   ONESHOT  every rank loads every peer's staging buffer and reduces all of
//            it: one barrier before the loads, latency-optimal.
//   TWOSHOT  rank r reduces chunk r from all peers (peer loads) and stores
//            the result into every peer's staging buffer (peer stores).
//   NVLS     same decomposition, but multimem.ld_reduce sums the chunk inside
//            the NVSwitch and multimem.st broadcasts it.
// CTA b of one rank only ever depends on CTA b of the other ranks (the data
// is partitioned so that what CTA b reads from a peer was written by CTA b
// there), so no grid-wide synchronisation is needed.
#include "tensor_walk.cuh"

namespace hvd {
namespace kern {

namespace {

constexpr int THREADS = 512;

template <typename T, typename W, typename S, int UNROLL = 4>
__device__ __forceinline__ void pack_range(const TensorList& tl, uint4* stage,
                                           int64_t lo, int64_t hi, S scale,
                                           bool do_scale) {
  gather_range<T, W, S, THREADS, UNROLL>(tl, lo, hi, scale, do_scale,
                                 [stage](int64_t v, uint4 x) { st16(stage + v, x); });
}

template <typename T, typename W, typename S>
__device__ __forceinline__ void unpack_range(const TensorList& tl,
                                             const uint4* stage, int64_t lo,
                                             int64_t hi, S scale, bool do_scale) {
  scatter_range<T, W, S, THREADS>(tl, lo, hi, scale, do_scale,
                                  [stage](int64_t v) { return ld16(stage + v); });
}

// Sum of chunk vectors [lo, hi) over all ranks by peer loads, result stored
// into every rank's staging buffer. WORLD is a compile-time copy of
// ctx.world so that the loads of several vectors are all issued before the
// first add (UNROLL vectors x WORLD peers in flight per thread).
template <typename W, int WORLD, int UNROLL>
__device__ __forceinline__ void reduce_chunk_p2p(const SymmCtx& ctx, int64_t lo,
                                                 int64_t hi) {
  const int rank = ctx.rank;
  const uint4* src[WORLD];
  uint4* dst[WORLD];
#pragma unroll
  for (int i = 0; i < WORLD; ++i) {
    // Start at a different peer on every rank to spread the load.
    int p = rank + i;
    if (p >= WORLD) p -= WORLD;
    src[i] = reinterpret_cast<const uint4*>(ctx.peers[p]);
    dst[i] = reinterpret_cast<uint4*>(ctx.peers[p]);
  }
  int64_t v = lo + threadIdx.x;
  for (; v + (UNROLL - 1) * THREADS < hi; v += UNROLL * THREADS) {
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
      const uint4 sum = acc.pack();
#pragma unroll
      for (int i = 0; i < WORLD; ++i) st16(dst[i] + v + u * THREADS, sum);
    }
  }
  for (; v < hi; v += THREADS) {
    VecAcc<W> acc;
    acc.zero();
#pragma unroll
    for (int i = 0; i < WORLD; ++i) acc.add(ld16(src[i] + v));
    const uint4 sum = acc.pack();
#pragma unroll
    for (int i = 0; i < WORLD; ++i) st16(dst[i] + v, sum);
  }
}

// One-shot: every rank sums vectors [lo, hi) of all ranks' staging buffers
// and scatters the result straight into its own output tensors. The adds run
// in rank order on every GPU, so all ranks compute bitwise-identical sums.
template <typename T, typename W, typename S, int WORLD, int UNROLL>
__device__ __forceinline__ void oneshot_reduce(const TensorList& tl, const SymmCtx& ctx,
                                               int64_t lo, int64_t hi, S postscale,
                                               bool post) {
  const uint4* src[WORLD];
#pragma unroll
  for (int p = 0; p < WORLD; ++p) src[p] = reinterpret_cast<const uint4*>(ctx.peers[p]);
  scatter_range<T, W, S, THREADS, UNROLL>(tl, lo, hi, postscale, post, [&](int64_t v) {
    uint4 in[WORLD];
#pragma unroll
    for (int p = 0; p < WORLD; ++p) in[p] = ld16(src[p] + v);
    VecAcc<W> acc;
    acc.zero();
#pragma unroll
    for (int p = 0; p < WORLD; ++p) acc.add(in[p]);
    return acc.pack();
  });
}

// INLINE: the tensor list rides in the kernel parameters (`inl`) and is
// copied to shared memory first (parameter reads with compile-time offsets
// only); else it is read from device memory (`tl_dev`).
template <typename T, typename W, int ALGO, bool INLINE>
__device__ __forceinline__ void fused_allreduce_body(const InlineTensors& inl,
                                                     const TensorList& tl_dev,
                                                     const SymmCtx& ctx,
                                                     typename ScaleT<T>::type prescale,
                                                     typename ScaleT<T>::type postscale) {
  using S = typename ScaleT<T>::type;
  constexpr int N = 16 / sizeof(W);
  __shared__ int64_t s_offsets[INLINE ? INLINE_TENSORS + 1 : 1];
  __shared__ int64_t s_counts[INLINE ? INLINE_TENSORS : 1];
  __shared__ const void* s_in[INLINE ? INLINE_TENSORS : 1];
  __shared__ void* s_out[INLINE ? INLINE_TENSORS : 1];
  TensorList tl = tl_dev;
  if constexpr (INLINE) {
#pragma unroll
    for (int i = 0; i < INLINE_TENSORS; ++i) {
      if (threadIdx.x == i && i < inl.n) {
        s_offsets[i] = inl.offsets[i];
        s_counts[i] = inl.counts[i];
        s_in[i] = inl.in[i];
        s_out[i] = inl.out[i];
      }
    }
#pragma unroll
    for (int i = 1; i <= INLINE_TENSORS; ++i)
      if (threadIdx.x == 32 && i == inl.n) s_offsets[i] = inl.offsets[i];
    __syncthreads();
    tl.n = inl.n;
    tl.offsets = s_offsets;
    tl.counts = s_counts;
    tl.in = s_in;
    tl.out = s_out;
  }
  trace_mark(ctx, 0);
  const int64_t nvec = tl.offsets[tl.n] / N;
  const int world = ctx.world, rank = ctx.rank;
  const int G = gridDim.x, b = blockIdx.x;
  const bool pre = prescale != S(1), post = postscale != S(1);
  uint4* stage = reinterpret_cast<uint4*>(ctx.local);

  if constexpr (ALGO == static_cast<int>(Algo::LOCAL)) {
    const int64_t per = (nvec + G - 1) / G;
    const int64_t lo = b * per, hi = min(lo + per, nvec);
    // No staging on a single rank: gather (scale, round through the wire
    // type) and write straight back to the outputs.
    int cout = lo < hi ? find_tensor(tl, lo * N) : 0;
    // Same arithmetic as the multi-rank variants: prescale, round to the
    // wire type, postscale.
    gather_range<T, W, S, THREADS>(
        tl, lo, hi, prescale, pre, [&](int64_t v, uint4 x) {
          // Vectors arrive in increasing order per thread only inside one
          // tensor; re-seek when the walker moved on to the next tensor.
          if (v * N < tl.offsets[cout]) cout = find_tensor(tl, v * N);
          scatter_vec<T, W, S>(tl, cout, v * N, x, postscale, post);
        });
    return;
  } else if constexpr (ALGO == static_cast<int>(Algo::ONESHOT)) {
    const int64_t per = (nvec + G - 1) / G;
    const int64_t lo = b * per, hi = min(lo + per, nvec);
    pack_range<T, W, S>(tl, stage, lo, hi, prescale, pre);
    trace_mark(ctx, 1);
    if (!cta_barrier(ctx, ctx.epoch + 1, b, 1)) return;
    trace_mark(ctx, 2);
    switch (world) {
    case 2: oneshot_reduce<T, W, S, 2, 4>(tl, ctx, lo, hi, postscale, post); break;
    case 3: oneshot_reduce<T, W, S, 3, 2>(tl, ctx, lo, hi, postscale, post); break;
    case 4: oneshot_reduce<T, W, S, 4, 2>(tl, ctx, lo, hi, postscale, post); break;
    case 5: oneshot_reduce<T, W, S, 5, 1>(tl, ctx, lo, hi, postscale, post); break;
    case 6: oneshot_reduce<T, W, S, 6, 1>(tl, ctx, lo, hi, postscale, post); break;
    case 7: oneshot_reduce<T, W, S, 7, 1>(tl, ctx, lo, hi, postscale, post); break;
    default: oneshot_reduce<T, W, S, 8, 1>(tl, ctx, lo, hi, postscale, post); break;
    }
    // Nobody may repack its staging buffer while a peer still reads it
    // (unless the caller alternates between two staging regions).
    trace_mark(ctx, 3);
    if (!ctx.skip_end_barrier) cta_barrier(ctx, ctx.epoch + 2, b, 2);
    trace_mark(ctx, 4);
    return;
  } else {
    // Two-shot / NVLS, software-pipelined over sub-chunks: CTA b owns slice b
    // of every rank's chunk and walks it in K steps. In step k it packs
    // sub-chunk k (of all `world` rank chunks) and announces it, reduces
    // sub-chunk k - 1 of its own rank's chunk once every peer has announced
    // that one, writes the sums into everybody's staging buffer and announces
    // them, and unpacks sub-chunk k - 2 once every peer has announced its
    // sums. Packing and unpacking (local HBM traffic) thereby overlap the
    // reduction (NVLink traffic) of the neighbouring sub-chunks. Two counters
    // per (rank, CTA) carry the announcements: "packed" in flag bank 0,
    // "reduced" in bank 3, both counting from ctx.epoch. After the last wait
    // nobody reads or writes this rank's staging buffer any more, so no
    // trailing barrier is needed; the launch consumes K + 1 epochs.
    constexpr int REDUCED_BANK = 3 * SYMM_MAX_RANKS * SYMM_MAX_BLOCKS;
    const int64_t per_rank = (nvec + world - 1) / world;
    const int64_t per_cta = (per_rank + G - 1) / G;
    const int64_t C = ctx.sub_chunk_vecs > 0 ? ctx.sub_chunk_vecs : per_cta;
    const int64_t K = max(int64_t(1), (per_cta + C - 1) / C);
    auto announce = [&](int bank, uint32_t value) {
      __syncthreads();
      if (threadIdx.x < world)
        st_release_sys(ctx.flags_peers[threadIdx.x] + bank + rank * SYMM_MAX_BLOCKS + b, value);
    };
    auto await = [&](int bank, uint32_t value, int phase) {
      bool ok = true;
      if (threadIdx.x < world) {
        const uint32_t* f = ctx.flags_local + bank + threadIdx.x * SYMM_MAX_BLOCKS + b;
        const unsigned long long t0 = globaltimer_ns();
        int spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - value) < 0) {
          if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
            ok = false;
            volatile int* st = ctx.status;
            st[1] = threadIdx.x;
            st[2] = phase;
            st[3] = b;
            __threadfence_system();
            if (st[0] == 0) st[0] = 1;
            __threadfence_system();
            break;
          }
        }
      }
      return __syncthreads_and(ok) != 0;
    };
    // Vector range of sub-chunk k inside rank r's chunk, for this CTA.
    auto sub = [&](int r, int64_t k, int64_t* lo, int64_t* hi) {
      const int64_t base = r * per_rank + b * per_cta;
      const int64_t end = min(base + per_cta, min((r + 1) * per_rank, nvec));
      *lo = min(end, base + k * C);
      *hi = min(end, base + (k + 1) * C);
    };
    for (int64_t k = 0; k < K + 2; ++k) {
      if (k < K) {
        for (int r = 0; r < world; ++r) {
          int64_t lo, hi;
          sub(r, k, &lo, &hi);
          pack_range<T, W, S>(tl, stage, lo, hi, prescale, pre);
        }
        announce(0, ctx.epoch + static_cast<uint32_t>(k) + 1u);
        if (k == K - 1) trace_mark(ctx, 1);
      }
      if (k >= 1 && k <= K) {
        if (!await(0, ctx.epoch + static_cast<uint32_t>(k), 1)) return;
        if (k == 1) trace_mark(ctx, 2);
        int64_t lo, hi;
        sub(rank, k - 1, &lo, &hi);
        if constexpr (ALGO == static_cast<int>(Algo::NVLS)) {
          uint4* mc = reinterpret_cast<uint4*>(ctx.mc);
          int64_t v = lo + threadIdx.x;
          for (; v + 3 * THREADS < hi; v += 4 * THREADS) {
            uint4 x0 = Multimem<W>::ld_reduce(mc + v);
            uint4 x1 = Multimem<W>::ld_reduce(mc + v + THREADS);
            uint4 x2 = Multimem<W>::ld_reduce(mc + v + 2 * THREADS);
            uint4 x3 = Multimem<W>::ld_reduce(mc + v + 3 * THREADS);
            multimem_st16(mc + v, x0);
            multimem_st16(mc + v + THREADS, x1);
            multimem_st16(mc + v + 2 * THREADS, x2);
            multimem_st16(mc + v + 3 * THREADS, x3);
          }
          for (; v < hi; v += THREADS)
            multimem_st16(mc + v, Multimem<W>::ld_reduce(mc + v));
        } else {
          switch (world) {
          case 2: reduce_chunk_p2p<W, 2, 4>(ctx, lo, hi); break;
          case 3: reduce_chunk_p2p<W, 3, 2>(ctx, lo, hi); break;
          case 4: reduce_chunk_p2p<W, 4, 2>(ctx, lo, hi); break;
          case 5: reduce_chunk_p2p<W, 5, 1>(ctx, lo, hi); break;
          case 6: reduce_chunk_p2p<W, 6, 1>(ctx, lo, hi); break;
          case 7: reduce_chunk_p2p<W, 7, 1>(ctx, lo, hi); break;
          default: reduce_chunk_p2p<W, 8, 1>(ctx, lo, hi); break;
          }
        }
        announce(REDUCED_BANK, ctx.epoch + static_cast<uint32_t>(k));
        if (k == K) trace_mark(ctx, 3);
      }
      if (k >= 2) {
        if (!await(REDUCED_BANK, ctx.epoch + static_cast<uint32_t>(k) - 1u, 2)) return;
        if (k == K + 1) trace_mark(ctx, 4);
        for (int r = 0; r < world; ++r) {
          int64_t lo, hi;
          sub(r, k - 2, &lo, &hi);
          unpack_range<T, W, S>(tl, stage, lo, hi, postscale, post);
        }
      }
    }
    trace_mark(ctx, 5);
  }
}

template <typename T, typename W, int ALGO, bool INLINE>
__global__ void __launch_bounds__(THREADS)
fused_allreduce_kernel(const InlineTensors inl, const TensorList tl_dev,
                       SymmCtx ctx, typename ScaleT<T>::type prescale,
                       typename ScaleT<T>::type postscale) {
  fused_allreduce_body<T, W, ALGO, INLINE>(inl, tl_dev, ctx, prescale, postscale);
}

// Stands in for the inline list of the variant that does not read it.
__device__ InlineTensors g_no_inline_list;

// Several ranks on one GPU (tests): one cooperative launch whose grid is
// (CTAs per rank, ranks); row y runs the kernel of rank y with that rank's
// tensor list and context, so the rows can wait for one another like the
// kernels of different GPUs do.
template <typename T, typename W, int ALGO>
__global__ void __launch_bounds__(THREADS)
fused_allreduce_emulated_kernel(const EmuAllreduceRank* ranks,
                                typename ScaleT<T>::type prescale,
                                typename ScaleT<T>::type postscale) {
  const EmuAllreduceRank& r = ranks[blockIdx.y];
  fused_allreduce_body<T, W, ALGO, false>(g_no_inline_list, r.tl, r.ctx, prescale, postscale);
}

template <typename T, typename W, bool INLINE>
cudaError_t LaunchAlgo(const InlineTensors& inl, const TensorList& tl, Algo algo,
                       int num_ctas, const SymmCtx& ctx, cudaStream_t stream,
                       typename ScaleT<T>::type pre, typename ScaleT<T>::type post) {
  switch (algo) {
  case Algo::LOCAL:
    fused_allreduce_kernel<T, W, 0, INLINE><<<num_ctas, THREADS, 0, stream>>>(inl, tl, ctx, pre, post);
    break;
  case Algo::ONESHOT:
    fused_allreduce_kernel<T, W, 1, INLINE><<<num_ctas, THREADS, 0, stream>>>(inl, tl, ctx, pre, post);
    break;
  case Algo::TWOSHOT:
    fused_allreduce_kernel<T, W, 2, INLINE><<<num_ctas, THREADS, 0, stream>>>(inl, tl, ctx, pre, post);
    break;
  case Algo::NVLS:
    if constexpr (std::is_same<W, float>::value || std::is_same<W, __half>::value ||
                  std::is_same<W, __nv_bfloat16>::value) {
      if (ctx.mc == nullptr) return cudaErrorInvalidValue;
      fused_allreduce_kernel<T, W, 3, INLINE><<<num_ctas, THREADS, 0, stream>>>(inl, tl, ctx, pre, post);
    } else {
      return cudaErrorInvalidValue;
    }
    break;
  }
  return cudaGetLastError();
}

template <typename T, typename W>
cudaError_t LaunchTyped(const TensorList& tl, double prescale, double postscale,
                        Algo algo, int num_ctas, const SymmCtx& ctx,
                        cudaStream_t stream, const InlineTensors* inline_list) {
  using S = typename ScaleT<T>::type;
  const S pre = static_cast<S>(prescale), post = static_cast<S>(postscale);
  static const InlineTensors kNoInline = {};
  if (inline_list != nullptr && inline_list->n > 0)
    return LaunchAlgo<T, W, true>(*inline_list, tl, algo, num_ctas, ctx, stream, pre, post);
  return LaunchAlgo<T, W, false>(kNoInline, tl, algo, num_ctas, ctx, stream, pre, post);
}

template <typename T, typename W>
cudaError_t LaunchEmulatedTyped(const EmuAllreduceRank* ranks, int world, double prescale,
                                double postscale, Algo algo, int num_ctas,
                                cudaStream_t stream) {
  using S = typename ScaleT<T>::type;
  S pre = static_cast<S>(prescale), post = static_cast<S>(postscale);
  void* args[] = {&ranks, &pre, &post};
  const dim3 grid(num_ctas, world);
  const void* fn = nullptr;
  if (algo == Algo::ONESHOT)
    fn = reinterpret_cast<const void*>(&fused_allreduce_emulated_kernel<T, W, 1>);
  else if (algo == Algo::TWOSHOT)
    fn = reinterpret_cast<const void*>(&fused_allreduce_emulated_kernel<T, W, 2>);
  else
    return cudaErrorInvalidValue;  // multimem needs a multicast object over several GPUs
  // Cooperative: fails instead of deadlocking when the rows do not all fit on
  // the GPU at once.
  return cudaLaunchCooperativeKernel(fn, grid, dim3(THREADS), args, 0, stream);
}

}  // namespace

cudaError_t LaunchFusedAllreduceEmulated(const EmuAllreduceRank* ranks, int world,
                                         DataType dtype, DataType wire, double prescale,
                                         double postscale, Algo algo, int num_ctas,
                                         cudaStream_t stream) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS || world < 1 || world > SYMM_MAX_RANKS)
    return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  if (dtype == DataType::FLOAT32 && wire == DataType::BFLOAT16)
    return LaunchEmulatedTyped<float, __nv_bfloat16>(ranks, world, prescale, postscale, algo,
                                                     num_ctas, stream);
  if (dtype != wire) return cudaErrorInvalidValue;
  switch (dtype) {
  case DataType::FLOAT32:
    return LaunchEmulatedTyped<float, float>(ranks, world, prescale, postscale, algo, num_ctas,
                                             stream);
  case DataType::BFLOAT16:
    return LaunchEmulatedTyped<__nv_bfloat16, __nv_bfloat16>(ranks, world, prescale, postscale,
                                                             algo, num_ctas, stream);
  case DataType::INT32:
    return LaunchEmulatedTyped<int32_t, int32_t>(ranks, world, prescale, postscale, algo,
                                                 num_ctas, stream);
  default:
    return cudaErrorInvalidValue;
  }
}

cudaError_t LaunchFusedAllreduce(const TensorList& tl, DataType dtype,
                                 DataType wire, double prescale,
                                 double postscale, Algo algo, int num_ctas,
                                 const SymmCtx& ctx, cudaStream_t stream,
                                 const InlineTensors* inline_list) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  if (dtype == DataType::FLOAT32 && wire == DataType::BFLOAT16)
    return LaunchTyped<float, __nv_bfloat16>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  if (dtype == DataType::FLOAT32 && wire == DataType::FLOAT16)
    return LaunchTyped<float, __half>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  if (dtype != wire) return cudaErrorInvalidValue;
  switch (dtype) {
  case DataType::FLOAT32:
    return LaunchTyped<float, float>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  case DataType::FLOAT16:
    return LaunchTyped<__half, __half>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  case DataType::BFLOAT16:
    return LaunchTyped<__nv_bfloat16, __nv_bfloat16>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  case DataType::FLOAT64:
    return LaunchTyped<double, double>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  case DataType::INT32:
    return LaunchTyped<int32_t, int32_t>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  case DataType::INT64:
    return LaunchTyped<int64_t, int64_t>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  case DataType::UINT8:
    return LaunchTyped<uint8_t, uint8_t>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  case DataType::INT8:
    return LaunchTyped<int8_t, int8_t>(tl, prescale, postscale, algo, num_ctas, ctx, stream, inline_list);
  default:
    return cudaErrorInvalidValue;
  }
}

}  // namespace kern
}  // namespace hvd
