// Pipelined variant of the exchange kernel (allgather / broadcast / alltoall
// through the peers' staging buffers) for large rounds: pushing chunks over
// NVLink and delivering received chunks into their final tensors overlap
// instead of running back to back around one barrier.
//
// CTA b of rank r walks its outbound segments in plan order, slice b of each,
// in chunks of plan.chunk_bytes. After every chunk it publishes its running
// chunk count n as the value ctx.epoch + n in the flag word [r][b] of every
// peer (release store after a CTA barrier, so the chunk's bytes are visible
// first). Between two pushes, and after the last one, it delivers inbound
// chunks: chunk k of inbound segment s (written by CTA b of rank
// in_src_rank[s]) is ready once that flag word has reached
// ctx.epoch + in_wait_base[s] + k + 1. While the CTA still has chunks to push
// the check does not block; afterwards it is a bounded spin. The trailing
// barrier (value ctx.epoch + plan.done_epochs) keeps peers from reusing this
// staging buffer before it has been drained.
//
// Selected by HOROVOD_EXCHANGE_PIPELINE=1 for rounds of 8 MiB and more; the
// two-phase kernel in exchange.cu stays the default.
#include "exchange_common.cuh"

namespace hvd {
namespace kern {

namespace {

using namespace exch;

// All threads call it. Thread 0 waits (bounded) until the flag word of
// (source rank, this CTA) has reached `want`; false after a timeout, with the
// status record naming the peer.
__device__ __forceinline__ bool wait_progress(const SymmCtx& ctx, int src, int block,
                                              uint32_t want, int phase) {
  bool ok = true;
  if (threadIdx.x == 0) {
    const uint32_t* f = ctx.flags_local + src * SYMM_MAX_BLOCKS + block;
    const unsigned long long t0 = globaltimer_ns();
    int spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - want) < 0) {
      if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
        ok = false;
        volatile int* st = ctx.status;
        st[1] = src;
        st[2] = phase;
        st[3] = block;
        __threadfence_system();
        if (st[0] == 0) st[0] = 1;
        __threadfence_system();
        break;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

__global__ void __launch_bounds__(THREADS)
exchange_pipelined_kernel(const PipelinePlan plan, SymmCtx ctx) {
  const int b = blockIdx.x, G = gridDim.x;
  const int64_t C = plan.chunk_bytes;
  __shared__ int s_ready;

  int so = 0, si = 0;      // current outbound / inbound segment
  int64_t ko = 0, ki = 0;  // current chunk inside it
  uint32_t published = 0;  // chunks this CTA has made visible so far

  for (;;) {
    // ---- push one chunk ----------------------------------------------------
    if (so < plan.n_out) {
      const int64_t off = plan.out_staging_off[so], bytes = plan.out_bytes[so];
      const int64_t K = ExchangeChunkCount(bytes, G, C);
      int64_t lo, hi;
      my_range(off, bytes, b, G, &lo, &hi);
      const int64_t clo = lo + ko * C, chi = min(hi, clo + C);
      if (clo < chi) {
        const char* src = static_cast<const char*>(plan.out_src[so]) + clo;
        const int dst_rank = plan.out_dst_rank[so];
        if (dst_rank >= 0) {
          copy_bytes(src, ctx.peers[dst_rank] + off + clo, chi - clo, TO_PEER, ctx, off + clo);
        } else {
          copy_bytes(src, ctx.local + off + clo, chi - clo,
                     ctx.mc != nullptr ? TO_ALL_MC : TO_ALL_LOOP, ctx, off + clo);
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
    // ---- deliver every inbound chunk that has arrived ----------------------
    while (si < plan.n_in) {
      const int64_t off = plan.in_staging_off[si], bytes = plan.in_bytes[si];
      const int64_t K = ExchangeChunkCount(bytes, G, C);
      const int src_rank = plan.in_src_rank[si];
      const uint32_t want =
          ctx.epoch + static_cast<uint32_t>(plan.in_wait_base[si]) + static_cast<uint32_t>(ki) + 1u;
      if (threadIdx.x == 0)
        s_ready = static_cast<int32_t>(
                      ld_acquire_sys(ctx.flags_local + src_rank * SYMM_MAX_BLOCKS + b) - want) >= 0;
      __syncthreads();
      const bool ready = s_ready != 0;
      __syncthreads();  // s_ready is rewritten by the next check
      if (!ready) {
        if (so < plan.n_out) break;  // push more first, look again afterwards
        if (!wait_progress(ctx, src_rank, b, want, 3)) return;
      }
      int64_t lo, hi;
      my_range(off, bytes, b, G, &lo, &hi);
      const int64_t clo = lo + ki * C, chi = min(hi, clo + C);
      char* dst = static_cast<char*>(plan.in_dst[si]);
      if (dst != nullptr && clo < chi)
        copy_bytes(ctx.local + off + clo, dst + clo, chi - clo, LOCAL_COPY, ctx, 0);
      if (++ki == K) {
        ki = 0;
        ++si;
      }
    }
    if (so >= plan.n_out && si >= plan.n_in) break;
  }
  // Nobody reuses this staging buffer before everybody has drained it.
  cta_barrier(ctx, ctx.epoch + plan.done_epochs, b, 4);
}

}  // namespace

cudaError_t LaunchExchangePipelined(const PipelinePlan& plan, int num_ctas,
                                    const SymmCtx& ctx, cudaStream_t stream) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  if (plan.chunk_bytes < 4096 || (plan.chunk_bytes & 255) != 0) return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  exchange_pipelined_kernel<<<num_ctas, THREADS, 0, stream>>>(plan, ctx);
  return cudaGetLastError();
}

}  // namespace kern
}  // namespace hvd
