// Allgather, broadcast and alltoall as one "exchange" kernel: every outbound
// segment is copied from local tensor storage straight into the destination
// rank's staging buffer over NVLink (peer stores; a segment addressed to all
// ranks is written once through the multicast mapping with multimem.st when
// available), one cross-GPU barrier follows, and every inbound segment is
// copied from the local staging buffer into its final tensor.
//
// A segment is owned by the same CTA index on the sending and the receiving
// rank (small segments by a hash of their staging offset, large ones split
// evenly), so CTA b only waits for CTA b of its peers.
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

// INLINE: the plan rides in the kernel parameters and is copied to shared
// memory first (parameter reads with compile-time offsets only); else it is
// read from device memory.
template <bool INLINE>
__global__ void __launch_bounds__(THREADS)
exchange_kernel(const InlineExchange inl, const ExchangePlan plan_dev, SymmCtx ctx) {
  const int b = blockIdx.x, G = gridDim.x;
  constexpr int SEGS = INLINE ? INLINE_SEGMENTS : 1;
  __shared__ const void* s_out_src[SEGS];
  __shared__ int64_t s_out_off[SEGS];
  __shared__ int64_t s_out_bytes[SEGS];
  __shared__ int32_t s_out_rank[SEGS];
  __shared__ void* s_in_dst[SEGS];
  __shared__ int64_t s_in_off[SEGS];
  __shared__ int64_t s_in_bytes[SEGS];
  ExchangePlan plan = plan_dev;
  if constexpr (INLINE) {
#pragma unroll
    for (int i = 0; i < INLINE_SEGMENTS; ++i) {
      if (threadIdx.x == i && i < inl.n_out) {
        s_out_src[i] = inl.out_src[i];
        s_out_off[i] = inl.out_staging_off[i];
        s_out_bytes[i] = inl.out_bytes[i];
        s_out_rank[i] = inl.out_dst_rank[i];
      }
      if (threadIdx.x == 32 + i && i < inl.n_in) {
        s_in_dst[i] = inl.in_dst[i];
        s_in_off[i] = inl.in_staging_off[i];
        s_in_bytes[i] = inl.in_bytes[i];
      }
    }
    __syncthreads();
    plan.n_out = inl.n_out;
    plan.out_src = s_out_src;
    plan.out_staging_off = s_out_off;
    plan.out_bytes = s_out_bytes;
    plan.out_dst_rank = s_out_rank;
    plan.n_in = inl.n_in;
    plan.in_dst = s_in_dst;
    plan.in_staging_off = s_in_off;
    plan.in_bytes = s_in_bytes;
  }
  for (int s = 0; s < plan.n_out; ++s) {
    const int64_t off = plan.out_staging_off[s], bytes = plan.out_bytes[s];
    int64_t lo, hi;
    my_range(off, bytes, b, G, &lo, &hi);
    if (lo >= hi) continue;
    const char* src = static_cast<const char*>(plan.out_src[s]) + lo;
    const int dst_rank = plan.out_dst_rank[s];
    if (dst_rank >= 0) {
      copy_bytes(src, ctx.peers[dst_rank] + off + lo, hi - lo, TO_PEER, ctx, off + lo);
    } else {
      copy_bytes(src, ctx.local + off + lo, hi - lo,
                 ctx.mc != nullptr ? TO_ALL_MC : TO_ALL_LOOP, ctx, off + lo);
    }
  }
  if (!cta_barrier(ctx, ctx.epoch + 1, b, 1)) return;
  for (int s = 0; s < plan.n_in; ++s) {
    const int64_t off = plan.in_staging_off[s], bytes = plan.in_bytes[s];
    int64_t lo, hi;
    my_range(off, bytes, b, G, &lo, &hi);
    if (lo >= hi) continue;
    char* dst = static_cast<char*>(plan.in_dst[s]);
    if (dst == nullptr) continue;
    copy_bytes(ctx.local + off + lo, dst + lo, hi - lo, LOCAL_COPY, ctx, 0);
  }
  // Keep peers from overwriting this staging buffer with their next
  // exchange before it has been drained.
  cta_barrier(ctx, ctx.epoch + 2, b, 2);
}

__global__ void barrier_only_kernel(SymmCtx ctx) {
  cta_barrier(ctx, ctx.epoch + 1, blockIdx.x, 1);
}

}  // namespace

cudaError_t LaunchExchange(const ExchangePlan& plan, int num_ctas,
                           const SymmCtx& ctx, cudaStream_t stream,
                           const InlineExchange* inline_plan) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  static const InlineExchange kNoInline = {};
  if (inline_plan != nullptr && (inline_plan->n_out > 0 || inline_plan->n_in > 0))
    exchange_kernel<true><<<num_ctas, THREADS, 0, stream>>>(*inline_plan, plan, ctx);
  else
    exchange_kernel<false><<<num_ctas, THREADS, 0, stream>>>(kNoInline, plan, ctx);
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
