// Host-side launch API of the sm_100a collective kernels. Every kernel works
// on symmetric memory (see symm/symm_arena.h): data moves between GPUs by
// loads/stores on peer pointers or by `multimem` instructions on the
// multicast mapping, issued from inside the kernel. Cross-GPU
// synchronisation uses per-(rank, CTA) flag words with release/acquire
// semantics and a monotonically increasing epoch; every wait is bounded and
// reports a timeout through a host-visible status record instead of hanging.
//
// These kernels replace the reference's pack -> NCCL -> unpack sequences
// (horovod/common/ops/nccl_operations.cc:156-727 and
// horovod/common/ops/cuda/cuda_kernels.cu:44-321).
#pragma once

#include <cstdint>

#include <cuda_runtime_api.h>

#include "../common/common.h"
#include "../symm/symm_arena.h"

namespace hvd {
namespace kern {

// Kernel-side view of the symmetric arena for one launch.
struct SymmCtx {
  int rank;
  int world;
  char* local;
  char* peers[SYMM_MAX_RANKS];
  char* mc;  // null when multicast is unavailable
  uint32_t* flags_local;
  uint32_t* flags_peers[SYMM_MAX_RANKS];
  uint32_t epoch;  // flags of this launch take values epoch+1, epoch+2, ...
  unsigned long long timeout_ns;
  int* status;  // host-mapped KernelStatus
  // When non-zero the kernel may skip its trailing barrier: the caller
  // guarantees that the staging region used by this launch is not written
  // again before every peer has passed a later barrier (double buffering).
  int skip_end_barrier;
  // Two-shot / NVLS fused allreduce: 16-byte vectors per pipeline step of one
  // CTA inside one rank's chunk (0 = no pipelining: one step). The launch
  // consumes ceil(per-CTA slice / sub_chunk_vecs) + 1 epochs.
  int64_t sub_chunk_vecs;
  // Optional phase timestamps (HOROVOD_KERNEL_TRACE=1): thread 0 of CTA 0
  // stores %globaltimer into trace[slot] at the kernel's phase boundaries.
  unsigned long long* trace;
};
constexpr int KERNEL_TRACE_SLOTS = 8;

// Written by a kernel whose bounded wait ran out. code 0 = fine.
struct KernelStatus {
  int code;   // 1 = timeout waiting for a peer flag, 2 = symmetric-tensor mismatch
  int peer;   // rank that never arrived
  int phase;  // which barrier inside the kernel
  int block;  // CTA that gave up
};

enum class Algo : int {
  LOCAL = 0,    // world == 1: scaled copy only
  ONESHOT = 1,  // every rank reads all peers and reduces the whole buffer
  TWOSHOT = 2,  // reduce-scatter by peer loads + allgather by peer stores
  NVLS = 3,     // multimem.ld_reduce + multimem.st through the switch
};

// Per-launch tensor list, in device memory. Tensor i occupies elements
// [offsets[i], offsets[i] + counts[i]) of the fused index space; offsets are
// multiples of 16 bytes of the wire type; offsets[n] is the padded total.
// A null input contributes zeros; a null output discards the result.
struct TensorList {
  int n;
  const int64_t* offsets;  // n + 1 entries
  const int64_t* counts;   // n entries
  const void* const* in;   // n entries
  void* const* out;        // n entries
};

// Small tensor lists travel inside the kernel's parameters instead of device
// memory, which saves the host-to-device descriptor copy in front of
// latency-bound launches.
constexpr int INLINE_TENSORS = 32;
struct InlineTensors {
  int n;  // 0 = not used, read the TensorList in device memory
  int64_t offsets[INLINE_TENSORS + 1];
  int64_t counts[INLINE_TENSORS];
  const void* in[INLINE_TENSORS];
  void* out[INLINE_TENSORS];
};

// Number of barrier epochs a launch of each kernel consumes (the pipelined
// two-shot / NVLS allreduce and the exchange kernels consume more: one per
// sub-chunk, see their launch code).
constexpr uint32_t EPOCHS_PER_LAUNCH = 4;
// Epochs of a two-shot / NVLS fused allreduce launch over `total_vecs`
// 16-byte vectors with `num_ctas` CTAs and `sub_chunk_vecs` per step.
inline uint32_t FusedAllreduceEpochs(int64_t total_vecs, int world, int num_ctas,
                                     int64_t sub_chunk_vecs) {
  const int64_t per_rank = (total_vecs + world - 1) / world;
  const int64_t per_cta = (per_rank + num_ctas - 1) / num_ctas;
  const int64_t k = sub_chunk_vecs > 0 ? (per_cta + sub_chunk_vecs - 1) / sub_chunk_vecs : 1;
  return static_cast<uint32_t>((k < 1 ? 1 : k) + 1);
}
// The Adasum driver launches 2 * log2(world) + 2 kernels, one epoch each.
constexpr uint32_t ADASUM_EPOCHS = 16;

// Fused multi-tensor allreduce (sum): gather from tensor storage with
// prescale and cast to the wire type, reduce across GPUs, postscale, cast
// back and scatter to the outputs, in one launch.
// dtype: element type of the tensors. wire: element type in the staging
// buffer and on NVLink (same as dtype, or FLOAT16/BFLOAT16 for FLOAT32
// tensors). Returns cudaErrorInvalidValue for unsupported combinations.
// `inline_list` (optional): the same list carried in the kernel parameters;
// when given, `tensors` is ignored.
cudaError_t LaunchFusedAllreduce(const TensorList& tensors, DataType dtype,
                                 DataType wire, double prescale,
                                 double postscale, Algo algo, int num_ctas,
                                 const SymmCtx& ctx, cudaStream_t stream,
                                 const InlineTensors* inline_list = nullptr);

// Several ranks on ONE GPU, for tests of the cross-rank protocols where only
// one GPU is available: the kernels of all "ranks" run as one cooperative
// launch (grid = CTAs per rank x ranks, rank = blockIdx.y), so that their CTAs
// are resident together and can wait for one another, which separate launches
// on one GPU could not guarantee. Every rank's context points at that rank's
// slice of one device allocation (staging, flags); `ranks` is an array of
// `world` entries in device memory. One-shot and two-shot only (multimem
// needs a multicast object over several GPUs).
struct EmuAllreduceRank {
  TensorList tl;  // arrays in device memory
  SymmCtx ctx;
};
cudaError_t LaunchFusedAllreduceEmulated(const EmuAllreduceRank* ranks, int world,
                                         DataType dtype, DataType wire, double prescale,
                                         double postscale, Algo algo, int num_ctas,
                                         cudaStream_t stream);

// In-place allreduce (sum, then scale) of byte ranges of the symmetric arena:
// range i covers bytes [byte_off[i], byte_off[i] + bytes[i]) of every rank's
// arena (offsets from the arena base, 16-byte aligned starts); vec_start is
// the running count of 16-byte vectors (a ragged tail counts as one), n + 1
// entries. No staging, no copies: see inplace_allreduce.cu.
struct RangeList {
  int n;
  const int64_t* vec_start;
  const int64_t* byte_off;
  const int64_t* bytes;
};
struct InlineRanges {
  int n;  // 0 = not used
  int64_t vec_start[INLINE_TENSORS + 1];
  int64_t byte_off[INLINE_TENSORS];
  int64_t bytes[INLINE_TENSORS];
};
// Dynamic work distribution for large in-place allreduces: CTAs draw tiles of
// `tile_vecs` 16-byte vectors from a device counter that only ever grows. A
// launch with T tiles and G CTAs consumes exactly T + G counter values starting
// at `base` (every CTA draws once more than it gets). counter == nullptr: static
// split, one slice per CTA.
struct TileSchedule {
  unsigned long long* counter;
  unsigned long long base;
  int tile_vecs;
};
cudaError_t LaunchInplaceAllreduce(const RangeList& ranges, DataType dtype,
                                   double scale, bool use_nvls, int num_ctas,
                                   const SymmCtx& ctx, cudaStream_t stream,
                                   const InlineRanges* inline_ranges = nullptr,
                                   const TileSchedule* schedule = nullptr);

// Fused reduce-scatter: like the first half of the two-shot allreduce; rank
// r's output receives elements [shard_begin[r], shard_begin[r+1]) of the
// single input tensor (element offsets; ragged shards allowed).
cudaError_t LaunchFusedReducescatter(const void* in, void* out, int64_t count,
                                     const int64_t* shard_begin_dev,
                                     DataType dtype, double prescale,
                                     double postscale, bool use_nvls,
                                     int num_ctas, const SymmCtx& ctx,
                                     cudaStream_t stream, int64_t sym_in_off = -1);
// sym_in_off >= 0: the input already lives in symmetric memory at that byte
// offset of every rank's arena (ctx.local/peers/mc must then point at the
// arena base, and every shard must start on a 16-byte boundary); the kernel
// skips staging and reduces straight out of the peers' tensors. prescale is
// ignored in that mode: fold it into postscale.

// Reduce-scatter of a tensor in ordinary memory by pushing shards into their
// owners' exchange regions (reducescatter_push.cu). One launch covers the
// window [win_lo, win_hi) of element offsets inside every shard; the region of
// every rank holds one slot of slot_bytes per sending rank. slice_vecs is the
// number of 16-byte vectors of a shard window each CTA handles (a multiple of
// 16, the same for all shards: derived from the largest one). The launch
// consumes ceil(slice_vecs * 16 / chunk_bytes) + 1 epochs. Region reuse is
// guarded by the same launch credits as the exchange kernel below.
struct RsPushArgs {
  int64_t shard_begin[SYMM_MAX_RANKS + 1];  // element offsets, world + 1 entries used
  int64_t win_lo, win_hi;
  int64_t slot_bytes;
  int64_t slice_vecs;
  int64_t chunk_bytes;
  uint32_t credit_wait, credit_post;
  unsigned long long* done_counter;
  unsigned long long done_target;
};
cudaError_t LaunchReducescatterPush(const void* in, void* out, const RsPushArgs& args,
                                    DataType dtype, double prescale, double postscale,
                                    int num_ctas, const SymmCtx& ctx, cudaStream_t stream);

// Several ranks on one GPU (see EmuAllreduceRank). Every rank needs its own
// done_counter word.
struct EmuRsPushRank {
  const void* in;
  void* out;
  RsPushArgs args;
  SymmCtx ctx;
};
cudaError_t LaunchReducescatterPushEmulated(const EmuRsPushRank* ranks, int world,
                                            DataType dtype, double prescale, double postscale,
                                            int num_ctas, cudaStream_t stream);

// The same for several tensors of one dtype in one launch (a fused
// reducescatter response): the whole shard of every tensor must fit a sender
// slot of the region (tensor t at byte slot_off, a multiple of 256). Rank p
// owns rows [p * base_rows + min(p, extra_rows), ...) of row_elems elements.
// The launch consumes total_chunks + 1 epochs, total_chunks being the sum over
// the tensors of ceil(slice_vecs * 16 / chunk_bytes).
struct RsGroupTensor {
  const void* in;
  void* out;           // this rank's shard
  int64_t base_rows, extra_rows, row_elems;
  int64_t slot_off;
  int64_t slice_vecs;  // 16-byte vectors of the largest shard per CTA, multiple of 16
};
struct RsGroupArgs {
  const RsGroupTensor* tensors;  // device-visible
  int n_tensors;
  uint32_t total_chunks;
  int64_t slot_bytes;
  int64_t chunk_bytes;
  uint32_t credit_wait, credit_post;
  unsigned long long* done_counter;
  unsigned long long done_target;
};
cudaError_t LaunchReducescatterPushGroup(const RsGroupArgs& args, DataType dtype, double prescale,
                                         double postscale, int num_ctas, const SymmCtx& ctx,
                                         cudaStream_t stream);

// Exchange kernel behind allgather, broadcast and alltoall. Every rank copies
// the data it owes to others from its tensors into an exchange region and
// publishes how far it has got; every receiver copies what it needs out of a
// region into its final tensor. Per staged segment the host picks the region:
//   * the sender's OWN region ("stage locally, pull remotely"): a local copy
//     at HBM speed, then the receiver pulls straight out of the owner's region
//     over NVLink into its final tensor. Data crosses NVLink once and lands in
//     its destination without a second local pass: the choice for large
//     messages;
//   * the RECEIVER's region (peer stores), or every rank's region at once
//     (multimem.st through the switch when multicast is available): the data
//     travels with the announcement instead of being fetched afterwards, one
//     NVLink crossing less on the critical path: the choice for small
//     messages and for a broadcast root with multicast (its NVLink egress is S
//     instead of (N-1) S).
//
// Progress is published per CTA: CTA b cuts its slice of every staged segment
// into chunks and, after each chunk, stores ctx.epoch + (chunks so far) into
// flag word [its rank][b] of every peer; CTA b of a receiver pulls chunk k of
// a segment once that word has reached ctx.epoch + pl_wait + k + 1, so staging
// and pulling overlap and a receiver waits only for the ranks it reads from
// (a broadcast is one-way: the root waits for nobody).
//
// Region reuse is guarded by credits instead of a trailing barrier: two
// regions alternate; the last CTA of a launch tells every peer "my launch
// number s is over" (credit_post), and a launch that is about to overwrite a
// region first checks that every peer has finished the launch that used it
// last (credit_wait; normally true already). credit_post == 0 selects a
// trailing barrier instead (process sets other than the global one).
struct ExchangePlan {
  int n_stage;
  const void* const* st_src;   // local source tensors
  void* const* st_self;        // also copy to this local destination (null = no)
  const int64_t* st_off;       // byte offset in the region; < 0: local copy to st_self only
  const int64_t* st_bytes;
  const int32_t* st_dst;       // whose region: -2 this rank's, -1 every other rank's, >= 0 that rank's
  int n_pull;
  void* const* pl_dst;         // local destination tensors
  const int64_t* pl_off;       // byte offset in the owner's region
  const int64_t* pl_bytes;
  const int32_t* pl_src;       // rank whose region holds the data
  const int32_t* pl_sig;       // rank whose progress counter announces it
  const int32_t* pl_wait;      // chunks that rank has published before this segment
};
// Short plans can ride in the kernel parameters (no descriptor copy).
constexpr int INLINE_SEGMENTS = 16;
struct InlineExchange {
  int n_stage, n_pull;  // both 0 = not used
  const void* st_src[INLINE_SEGMENTS];
  void* st_self[INLINE_SEGMENTS];
  int64_t st_off[INLINE_SEGMENTS];
  int64_t st_bytes[INLINE_SEGMENTS];
  int32_t st_dst[INLINE_SEGMENTS];
  void* pl_dst[INLINE_SEGMENTS];
  int64_t pl_off[INLINE_SEGMENTS];
  int64_t pl_bytes[INLINE_SEGMENTS];
  int32_t pl_src[INLINE_SEGMENTS];
  int32_t pl_sig[INLINE_SEGMENTS];
  int32_t pl_wait[INLINE_SEGMENTS];
};
struct ExchangeSync {
  int64_t chunk_bytes;      // multiple of 256
  uint32_t done_epochs;     // epochs this launch consumes (> chunks published by any CTA)
  uint32_t credit_wait;     // 0 = nothing to wait for
  uint32_t credit_post;     // 0 = end with a barrier instead
  unsigned long long* done_counter;  // device word counting finished CTAs (monotonic)
  unsigned long long done_target;    // its value once every CTA of this launch is through
};
// Chunks into which every CTA of a launch with `num_ctas` CTAs cuts its slice
// of a segment of `bytes` bytes (the same number for all CTAs of all ranks; a
// CTA whose slice is shorter publishes the remaining counts without copying).
#if defined(__CUDACC__)
__host__ __device__
#endif
inline int64_t ExchangeChunkCount(int64_t bytes, int num_ctas, int64_t chunk_bytes) {
  if (bytes <= 64 * 1024) return 1;  // small segments are owned by one CTA
  int64_t slice = (bytes + num_ctas - 1) / num_ctas;
  slice = (slice + 255) & ~int64_t(255);
  int64_t k = (slice + chunk_bytes - 1) / chunk_bytes;
  return k < 1 ? 1 : k;
}
cudaError_t LaunchExchange(const ExchangePlan& plan, const ExchangeSync& sync, int num_ctas,
                           const SymmCtx& ctx, cudaStream_t stream,
                           const InlineExchange* inline_plan = nullptr);

// Adasum over symmetric memory. Tensors are packed into staging as fp32
// (prescaled), combined pairwise over log2(world) levels with per-tensor
// dot / squared norms accumulated in fp64, and scattered back. `scratch`
// holds 3 * n doubles per level per rank inside the staging area (offset
// given in bytes, 256-byte aligned).
// copy_off >= 0: byte offset (256-byte aligned, inside the staging area) of
// room for half of the packed data: the partner's half is then copied there
// while the dot products read it, and the combine step reads the copy, so
// every level moves its data over NVLink once instead of twice.
cudaError_t LaunchAdasum(const TensorList& tensors, DataType dtype,
                         double prescale, double postscale,
                         int64_t scratch_off, int num_ctas, const SymmCtx& ctx,
                         cudaStream_t stream, int64_t copy_off = -1);

// Stand-alone helpers (NCCL path and odd cases).
// Batched (optionally scaled / casting) copy between tensor storage and a
// contiguous fusion buffer. to_buffer: tensors -> buffer, else the reverse.
// total_elements (the padded fused length) only sizes the grid.
cudaError_t LaunchPackUnpack(const TensorList& tensors, DataType dtype,
                             DataType wire, void* buffer, double scale,
                             bool to_buffer, int64_t total_elements,
                             cudaStream_t stream);
// out[i] = in[i] * scale for any dtype (integers scale in double).
cudaError_t LaunchScaleBuffer(const void* in, void* out, int64_t count,
                              DataType dtype, double scale,
                              cudaStream_t stream);

// Number of kernels of this library launched so far in this process (every
// Launch* function counts the kernels it enqueues).
// Training-mode batch normalisation on channels-last 16-bit activations
// ([rows, channels] row-major), fused with the residual add and the ReLU.
// `sums_zeroed` is a zero-filled scratch of 2 * channels doubles. Forward:
// y = act(bn(x) [+ residual]); also writes the batch mean / inverse standard
// deviation and updates the running statistics (when given). Backward: dx,
// optionally dresidual (= gradient through the ReLU), dweight, dbias.
bool BatchNormSupported(int64_t rows, int channels);
cudaError_t LaunchBatchNormForward(const void* x, const void* residual, void* y, int64_t rows,
                                   int channels, bool bf16, double* sums_zeroed,
                                   const float* weight, const float* bias, float eps,
                                   float momentum, float* save_mean, float* save_invstd,
                                   float* running_mean, float* running_var, bool relu,
                                   cudaStream_t stream);
cudaError_t LaunchBatchNormBackward(const void* dy, const void* y, const void* x, void* dx,
                                    void* dresidual, int64_t rows, int channels, bool bf16,
                                    double* sums_zeroed, const float* weight,
                                    const float* save_mean, const float* save_invstd,
                                    float* dweight, float* dbias, bool relu,
                                    cudaStream_t stream);

// 3x3 / stride 2 / padding 1 max pooling on channels-last 16-bit activations
// ([n, h, w, channels], channels a multiple of 8). Forward writes the maxima
// and one byte per output element naming the winning window position (0..8);
// backward gathers dy through those bytes into dx (every element written).
bool MaxPool3s2Supported(int channels);
cudaError_t LaunchMaxPool3s2Forward(const void* x, void* y, unsigned char* idx, int n, int h,
                                    int w, int channels, bool bf16, cudaStream_t stream);
cudaError_t LaunchMaxPool3s2Backward(const void* dy, const unsigned char* idx, void* dx, int n,
                                     int h, int w, int channels, bool bf16, cudaStream_t stream);

// Multi-tensor SGD step in one launch (torch.optim.SGD arithmetic: weight
// decay added to the gradient, momentum buffer b = momentum * b + (1 -
// dampening) * g, or b = g on the first step, optional Nesterov, then
// p -= lr * update). Tensor i has counts[i] fp32 elements at params[i],
// grads[i], bufs[i] (bufs may be null when momentum == 0); the three arrays of
// a tensor must share one memory layout. chunk_tensor / chunk_start (device
// arrays of n_chunks entries) cut the tensors into pieces of at most
// chunk_elems elements, one per CTA iteration.
struct SgdTensors {
  int n;
  float* const* params;
  const float* const* grads;
  float* const* bufs;
  const int64_t* counts;
  int n_chunks;
  const int32_t* chunk_tensor;
  const int64_t* chunk_start;
  int64_t chunk_elems;
};
cudaError_t LaunchFusedSgd(const SgdTensors& t, float lr, float momentum, float dampening,
                           float weight_decay, bool nesterov, bool first_step, bool maximize,
                           cudaStream_t stream);

uint64_t KernelLaunchCount();
void CountKernelLaunches(int n);

// Test hook: a kernel that runs one cross-GPU barrier and nothing else.
// Several ranks on one GPU (see EmuAllreduceRank): the plan arrays live in
// device memory; every rank needs its own done_counter word.
struct EmuExchangeRank {
  ExchangePlan plan;
  ExchangeSync sync;
  SymmCtx ctx;
};
cudaError_t LaunchExchangeEmulated(const EmuExchangeRank* ranks, int world, int num_ctas,
                                   cudaStream_t stream);

// Tells every peer that this rank no longer reads the exchange region of
// launch number `value` (the word the exchange kernel's credit wait polls).
// For rounds whose transfers are copy-engine copies queued on the stream
// before this launch.
cudaError_t LaunchCreditPost(uint32_t value, const SymmCtx& ctx, cudaStream_t stream);

cudaError_t LaunchBarrierOnly(int num_ctas, int bank, const SymmCtx& ctx,
                              cudaStream_t stream);

}  // namespace kern
}  // namespace hvd
