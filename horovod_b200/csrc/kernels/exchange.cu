// Allgather, broadcast and alltoall as one "stage locally, pull remotely"
// exchange kernel (the protocol is described at ExchangePlan in kernels.h).
//
// A segment is owned by the same CTA index on the staging and the pulling
// rank (small segments by a hash of their region offset, large ones split
// evenly), so CTA b only ever waits for CTA b of the ranks it reads from.
// Every wait is bounded: when it runs out the CTA records who it was waiting
// for in the status word and leaves, and so does the rest of the job.
//
// Replaces ncclAllGather / grouped ncclBroadcast / ncclBcast per tensor /
// grouped ncclSend+ncclRecv and the cudaMemcpyAsync loops around them
// (horovod/common/ops/nccl_operations.cc:468-727,
// horovod/common/ops/gpu_operations.cc:350-363).
#include "exchange_common.cuh"

namespace hvd {
namespace kern {

namespace {

using namespace exch;

// Flag bank that carries the region credits: word [rank r][0] of this bank in
// my pad = number of the last exchange launch rank r has completed.
constexpr int CREDIT_BANK = 2 * SYMM_MAX_RANKS * SYMM_MAX_BLOCKS;

__device__ __forceinline__ void report_timeout(const SymmCtx& ctx, int peer, int phase,
                                               int block) {
  volatile int* st = ctx.status;
  st[1] = peer;
  st[2] = phase;
  st[3] = block;
  __threadfence_system();
  if (st[0] == 0) st[0] = 1;
  __threadfence_system();
}

// Thread 0 waits (bounded) until flag word `f` has reached `want`; all
// threads call it and learn the outcome.
__device__ __forceinline__ bool wait_word(const SymmCtx& ctx, const uint32_t* f, uint32_t want,
                                          int peer, int phase, int block) {
  bool ok = true;
  if (threadIdx.x == 0) {
    const unsigned long long t0 = globaltimer_ns();
    int spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - want) < 0) {
      if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
        ok = false;
        report_timeout(ctx, peer, phase, block);
        break;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// INLINE: the plan rides in the kernel parameters and is copied to shared
// memory first (parameter reads with compile-time offsets only); else it is
// read from device memory.
template <bool INLINE>
__device__ __forceinline__ void exchange_body(const InlineExchange& inl,
                                              const ExchangePlan& plan_dev,
                                              const ExchangeSync& sync, const SymmCtx& ctx) {
  const int b = blockIdx.x, G = gridDim.x;
  constexpr int SEGS = INLINE ? INLINE_SEGMENTS : 1;
  __shared__ const void* s_st_src[SEGS];
  __shared__ void* s_st_self[SEGS];
  __shared__ int64_t s_st_off[SEGS];
  __shared__ int64_t s_st_bytes[SEGS];
  __shared__ int32_t s_st_dst[SEGS];
  __shared__ void* s_pl_dst[SEGS];
  __shared__ int64_t s_pl_off[SEGS];
  __shared__ int64_t s_pl_bytes[SEGS];
  __shared__ int32_t s_pl_src[SEGS];
  __shared__ int32_t s_pl_sig[SEGS];
  __shared__ int32_t s_pl_wait[SEGS];
  __shared__ int s_ready;
  ExchangePlan plan = plan_dev;
  if constexpr (INLINE) {
#pragma unroll
    for (int i = 0; i < INLINE_SEGMENTS; ++i) {
      if (threadIdx.x == i && i < inl.n_stage) {
        s_st_src[i] = inl.st_src[i];
        s_st_self[i] = inl.st_self[i];
        s_st_off[i] = inl.st_off[i];
        s_st_bytes[i] = inl.st_bytes[i];
        s_st_dst[i] = inl.st_dst[i];
      }
      if (threadIdx.x == 32 + i && i < inl.n_pull) {
        s_pl_dst[i] = inl.pl_dst[i];
        s_pl_off[i] = inl.pl_off[i];
        s_pl_bytes[i] = inl.pl_bytes[i];
        s_pl_src[i] = inl.pl_src[i];
        s_pl_sig[i] = inl.pl_sig[i];
        s_pl_wait[i] = inl.pl_wait[i];
      }
    }
    plan.n_stage = inl.n_stage;
    plan.st_src = s_st_src;
    plan.st_self = s_st_self;
    plan.st_off = s_st_off;
    plan.st_bytes = s_st_bytes;
    plan.st_dst = s_st_dst;
    plan.n_pull = inl.n_pull;
    plan.pl_dst = s_pl_dst;
    plan.pl_off = s_pl_off;
    plan.pl_bytes = s_pl_bytes;
    plan.pl_src = s_pl_src;
    plan.pl_sig = s_pl_sig;
    plan.pl_wait = s_pl_wait;
  }
  __syncthreads();

  if (ctx.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0)  // kernel entry
    *reinterpret_cast<volatile unsigned long long*>(ctx.trace + 5) = globaltimer_ns();
  // The region this launch writes may still be read by peers that are behind:
  // wait until each of them has finished the launch that used it last.
  if (sync.credit_wait != 0) {
    bool ok = true;
    if (threadIdx.x < ctx.world) {
      const uint32_t* f = ctx.flags_local + CREDIT_BANK + threadIdx.x * SYMM_MAX_BLOCKS;
      const unsigned long long t0 = globaltimer_ns();
      int spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys(f) - sync.credit_wait) < 0) {
        if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
          ok = false;
          report_timeout(ctx, threadIdx.x, 0, b);
          break;
        }
      }
    }
    if (__syncthreads_and(ok) == 0) return;
  }

  trace_mark(ctx, 0);
  const int64_t C = sync.chunk_bytes;
  int so = 0, si = 0;      // current staged / pulled segment
  int64_t ko = 0, ki = 0;  // current chunk inside it
  uint32_t published = 0;  // chunks this CTA has made visible so far
  bool staged_all = false;

  for (;;) {
    // ---- stage one chunk (or one whole local-only copy) --------------------
    if (so < plan.n_stage) {
      const int64_t off = plan.st_off[so], bytes = plan.st_bytes[so];
      const char* src = static_cast<const char*>(plan.st_src[so]);
      char* self = static_cast<char*>(plan.st_self[so]);
      if (off < 0) {
        // Local copy only (data this rank sends to itself): even split.
        int64_t slice = (bytes + G - 1) / G;
        slice = (slice + 255) & ~int64_t(255);
        const int64_t lo = min(bytes, b * slice), hi = min(bytes, lo + slice);
        if (lo < hi && self != nullptr)
          copy_bytes<4>(src + lo, false, nullptr, false, self + lo, hi - lo);
        ++so;
      } else {
        const int64_t K = ExchangeChunkCount(bytes, G, C);
        int64_t lo, hi;
        my_range(off, bytes, b, G, &lo, &hi);
        const int64_t clo = lo + ko * C, chi = min(hi, clo + C);
        if (clo < chi) {
          const int d = plan.st_dst[so];
          char* own = self != nullptr ? self + clo : nullptr;
          if (d == -1 && ctx.mc == nullptr) {
            // Every other rank's region, one peer after the other.
            for (int p = 0; p < ctx.world; ++p) {
              if (p == ctx.rank) continue;
              copy_bytes<4>(src + clo, false, ctx.peers[p] + off + clo, false, own, chi - clo);
              own = nullptr;
            }
          } else {
            char* region = d == -2 ? ctx.local : d >= 0 ? ctx.peers[d] : ctx.mc;
            copy_bytes<4>(src + clo, false, region + off + clo, d == -1, own, chi - clo);
          }
        }
        __syncthreads();
        ++published;
        if (threadIdx.x < ctx.world)
          st_release_sys(ctx.flags_peers[threadIdx.x] + ctx.rank * SYMM_MAX_BLOCKS + b,
                         ctx.epoch + published);
        if (++ko == K) {
          ko = 0;
          ++so;
        }
      }
    }
    // ---- pull one announced chunk, then go back to staging ------------------
    // (one for one, so that on every rank some CTAs are copying locally while
    // others are reading over NVLink; once nothing is left to stage, the rest
    // is pulled in order with blocking waits)
    bool pulled = false;
    while (si < plan.n_pull && !(pulled && so < plan.n_stage)) {
      const int64_t off = plan.pl_off[si], bytes = plan.pl_bytes[si];
      const int64_t K = ExchangeChunkCount(bytes, G, C);
      int64_t lo, hi;
      my_range(off, bytes, b, G, &lo, &hi);
      const int64_t clo = lo + ki * C, chi = min(hi, clo + C);
      char* dst = static_cast<char*>(plan.pl_dst[si]);
      if (dst != nullptr && clo < chi) {
        const int sig = plan.pl_sig[si];
        const uint32_t* f = ctx.flags_local + sig * SYMM_MAX_BLOCKS + b;
        const uint32_t want = ctx.epoch + static_cast<uint32_t>(plan.pl_wait[si]) +
                              static_cast<uint32_t>(ki) + 1u;
        if (threadIdx.x == 0)
          s_ready = static_cast<int32_t>(ld_acquire_sys(f) - want) >= 0;
        __syncthreads();
        const bool ready = s_ready != 0;
        __syncthreads();  // s_ready is rewritten by the next check
        if (!ready) {
          if (so < plan.n_stage) break;  // stage more first, look again afterwards
          if (!wait_word(ctx, f, want, sig, 3, b)) return;
        }
        copy_bytes<8>(ctx.peers[plan.pl_src[si]] + off + clo, true, nullptr, false, dst + clo,
                      chi - clo);
        pulled = true;
      }
      if (++ki == K) {
        ki = 0;
        ++si;
      }
    }
    if (so >= plan.n_stage && si >= plan.n_pull) break;
    if (so >= plan.n_stage && !staged_all) {
      staged_all = true;
      trace_mark(ctx, 1);  // everything staged and announced
    }
  }
  trace_mark(ctx, 2);

  if (sync.credit_post != 0) {
    // The last CTA of this rank to get here tells every peer that this
    // launch no longer reads anybody's region. (Every CTA's loads have
    // returned by now: their values were stored before the barrier below. No
    // fence is needed to order loads that have completed, and a fence here
    // would wait for the acknowledgement of every remote store first.)
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0)
      s_last = atomicAdd(sync.done_counter, 1ull) + 1ull == sync.done_target;
    __syncthreads();
    if (s_last != 0) {
      if (threadIdx.x < ctx.world)  // one store per peer, in parallel
        st_release_sys(ctx.flags_peers[threadIdx.x] + CREDIT_BANK + ctx.rank * SYMM_MAX_BLOCKS,
                       sync.credit_post);
      if (ctx.trace != nullptr && threadIdx.x == 0)  // when this rank's slowest CTA finished
        *reinterpret_cast<volatile unsigned long long*>(ctx.trace + 4) = globaltimer_ns();
    }
  } else {
    // Nobody rewrites its region before everybody has drained it.
    cta_barrier(ctx, ctx.epoch + sync.done_epochs, b, 4);
  }
  trace_mark(ctx, 3);
}

template <bool INLINE>
__global__ void __launch_bounds__(THREADS, 2)
exchange_kernel(const InlineExchange inl, const ExchangePlan plan_dev, const ExchangeSync sync,
                SymmCtx ctx) {
  exchange_body<INLINE>(inl, plan_dev, sync, ctx);
}

// Stands in for the inline plan of the variant that does not read it.
__device__ InlineExchange g_no_inline_plan;

// Several ranks on one GPU (tests): row y of a cooperative launch runs the
// kernel of rank y (see EmuAllreduceRank).
__global__ void __launch_bounds__(THREADS, 2)
exchange_emulated_kernel(const EmuExchangeRank* ranks) {
  const EmuExchangeRank& r = ranks[blockIdx.y];
  exchange_body<false>(g_no_inline_plan, r.plan, r.sync, r.ctx);
}

__global__ void credit_post_kernel(SymmCtx ctx, uint32_t value) {
  // The copies that read the peers' regions were queued on this stream before
  // this launch, so they have completed; one release store per peer.
  if (threadIdx.x < ctx.world)
    st_release_sys(ctx.flags_peers[threadIdx.x] + CREDIT_BANK + ctx.rank * SYMM_MAX_BLOCKS, value);
}

__global__ void barrier_only_kernel(SymmCtx ctx) {
  cta_barrier(ctx, ctx.epoch + 1, blockIdx.x, 1);
}

}  // namespace

cudaError_t LaunchExchange(const ExchangePlan& plan, const ExchangeSync& sync, int num_ctas,
                           const SymmCtx& ctx, cudaStream_t stream,
                           const InlineExchange* inline_plan) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  // A segment of up to 64 KB is one chunk of one CTA, so a chunk must hold it.
  if (sync.chunk_bytes < 64 * 1024 || (sync.chunk_bytes & 255) != 0) return cudaErrorInvalidValue;
  if (sync.credit_post != 0 && sync.done_counter == nullptr) return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  static const InlineExchange kNoInline = {};
  if (inline_plan != nullptr && (inline_plan->n_stage > 0 || inline_plan->n_pull > 0))
    exchange_kernel<true><<<num_ctas, THREADS, 0, stream>>>(*inline_plan, plan, sync, ctx);
  else
    exchange_kernel<false><<<num_ctas, THREADS, 0, stream>>>(kNoInline, plan, sync, ctx);
  return cudaGetLastError();
}

cudaError_t LaunchExchangeEmulated(const EmuExchangeRank* ranks, int world, int num_ctas,
                                   cudaStream_t stream) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS || world < 1 || world > SYMM_MAX_RANKS)
    return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  void* args[] = {&ranks};
  return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(&exchange_emulated_kernel),
                                     dim3(num_ctas, world), dim3(THREADS), args, 0, stream);
}

cudaError_t LaunchCreditPost(uint32_t value, const SymmCtx& ctx, cudaStream_t stream) {
  CountKernelLaunches(1);
  credit_post_kernel<<<1, 32, 0, stream>>>(ctx, value);
  return cudaGetLastError();
}

cudaError_t LaunchBarrierOnly(int num_ctas, int bank, const SymmCtx& ctx,
                              cudaStream_t stream) {
  (void)bank;  // the caller already pointed ctx.flags_* at the bank
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  barrier_only_kernel<<<num_ctas, 32, 0, stream>>>(ctx);
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace hvd
