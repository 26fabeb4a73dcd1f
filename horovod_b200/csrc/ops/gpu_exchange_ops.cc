// Broadcast, allgather and alltoall on device tensors, all expressed as
// segment lists for the exchange kernel: staged segments go from local
// tensors into this rank's exchange region, pulled segments go from the
// owner's region (over NVLink) straight into the final tensors.
#include <algorithm>
#include <cstring>

#include "../common/logging.h"
#include "../common/process_set.h"
#include "exchange_plan.h"
#include "gpu_internal.h"
#include "host_trace.h"

namespace hvd {

namespace {
constexpr int64_t STAGING_ALIGN = 256;
}

// One launch of the exchange kernel. Every rank derives the same numbers from
// the round's block list: the grid size, the chunks per block, how many chunks
// a source has published before each of its blocks, and the epochs the launch
// consumes (the largest chunk total of any rank, plus one for a final barrier).
void GpuOps::LaunchExchangeSegments(const std::vector<StageSeg>& stage,
                                    const std::vector<PullSeg>& pull, SymmSet& set,
                                    int64_t round_bytes,
                                    const std::vector<RoundBlock>& round,
                                    bool copy_engine) {
  if (copy_engine && set.xchg_bytes > 0) {
    // Large blocks: the kernel only stages this rank's blocks in its own
    // region (and copies what it keeps) and ends with the barrier over all
    // ranks; the copy engines then read the peers' regions into the final
    // tensors at full NVLink rate while the SMs are free, and a one-warp
    // launch returns the region credit once those copies are done.
    static const std::vector<PullSeg> kNoPulls;
    const uint32_t s = set.xchg_seq + 1;  // the number the staging launch takes
    LaunchExchangeKernel(stage, kNoPulls, set, round_bytes, round, /*post_credit=*/false);
    const int64_t region_off = set.xchg_off[s & 1];
    // Every rank starts with its right-hand neighbour and goes round, so at
    // any time each source is read by one peer (all ranks reading rank 0
    // first would share its NVLink egress).
    std::vector<PullSeg> ordered(pull);
    std::stable_sort(ordered.begin(), ordered.end(), [&](const PullSeg& a, const PullSeg& b) {
      return (a.src_rank - set.rank + set.world) % set.world <
             (b.src_rank - set.rank + set.world) % set.world;
    });
    for (const PullSeg& p : ordered) {
      if (p.dst == nullptr || p.bytes == 0) continue;
      cudaError_t e = cudaMemcpyAsync(p.dst, set.peers[p.src_rank] + region_off + p.off,
                                      static_cast<size_t>(p.bytes), cudaMemcpyDeviceToDevice,
                                      stream_);
      if (e != cudaSuccess)
        throw std::runtime_error(std::string("exchange peer copy failed: ") +
                                 cudaGetErrorString(e));
    }
    kern::SymmCtx ctx = MakeCtx(set, 0, region_off);
    cudaError_t e = kern::LaunchCreditPost(s, ctx, stream_);
    if (e != cudaSuccess)
      throw std::runtime_error(std::string("exchange credit launch failed: ") +
                               cudaGetErrorString(e));
    return;
  }
  LaunchExchangeKernel(stage, pull, set, round_bytes, round, /*post_credit=*/true);
}

// post_credit: the kernel's last CTA returns the region credit; otherwise the
// kernel ends with a barrier over all ranks and the caller returns the credit.
void GpuOps::LaunchExchangeKernel(const std::vector<StageSeg>& stage,
                                  const std::vector<PullSeg>& pull, SymmSet& set,
                                  int64_t round_bytes, const std::vector<RoundBlock>& round,
                                  bool post_credit) {
  const size_t ns = stage.size(), np = pull.size();
  // The grid size must be the same on every rank (CTA b meets CTA b of its
  // peers), so it is derived from the bytes of the whole round, which all
  // ranks know, not from this rank's share of them.
  const int ctas = PickCtas(round_bytes);
  // Larger rounds publish in larger chunks (fewer fences per byte).
  const int64_t chunk = (round_bytes >= (64 << 20) ? std::max<int64_t>(exchange_chunk_bytes_, 1 << 20)
                                                   : exchange_chunk_bytes_) / 256 * 256;
  const ExchangeRoundSync rsync = ComputeExchangeRoundSync(round, set.world, ctas, chunk);
  const std::vector<int64_t>& before = rsync.before;
  const int64_t most = static_cast<int64_t>(rsync.done_epochs) - 1;
  if (most + 1 > (int64_t(1) << 30))
    throw std::runtime_error("exchange round needs too many chunks");

  kern::ExchangeSync sync;
  std::memset(&sync, 0, sizeof(sync));
  sync.chunk_bytes = chunk;
  sync.done_epochs = static_cast<uint32_t>(most + 1);
  int64_t region_off = 0;
  if (set.xchg_bytes > 0) {
    // Alternate between the two regions; launch s may overwrite what launch
    // s - 2 left there once every peer has finished that launch.
    const uint32_t s = ++set.xchg_seq;
    region_off = set.xchg_off[s & 1];
    sync.credit_wait = s > 2 ? s - 2 : 0;
    if (post_credit) {
      sync.credit_post = s;
      sync.done_counter = xchg_done_counter_;
      xchg_done_base_ += static_cast<unsigned long long>(ctas);
      sync.done_target = xchg_done_base_;
    }
  }

  kern::ExchangePlan plan;
  std::memset(&plan, 0, sizeof(plan));
  cudaError_t err;
  if (inline_descriptors_ && ns <= kern::INLINE_SEGMENTS && np <= kern::INLINE_SEGMENTS &&
      (ns || np)) {
    // Short plan: carried in the kernel parameters.
    kern::InlineExchange inl;
    inl.n_stage = static_cast<int>(ns);
    inl.n_pull = static_cast<int>(np);
    for (size_t i = 0; i < ns; ++i) {
      inl.st_src[i] = stage[i].src;
      inl.st_self[i] = stage[i].self_dst;
      inl.st_off[i] = stage[i].off;
      inl.st_bytes[i] = stage[i].bytes;
      inl.st_dst[i] = stage[i].dst;
    }
    for (size_t i = 0; i < np; ++i) {
      inl.pl_dst[i] = pull[i].dst;
      inl.pl_off[i] = pull[i].off;
      inl.pl_bytes[i] = pull[i].bytes;
      inl.pl_src[i] = pull[i].src_rank;
      inl.pl_sig[i] = pull[i].sig_rank;
      inl.pl_wait[i] = static_cast<int32_t>(before[pull[i].block]);
    }
    kern::SymmCtx ctx = MakeCtx(set, sync.done_epochs, region_off);
    host_trace::Mark("plan");
    err = kern::LaunchExchange(plan, sync, ctas, ctx, stream_, &inl);
    host_trace::Mark("launch");
  } else {
    DescriptorRing::Slot slot = ring_.Acquire();
    const void** d_src;
    void **d_self, **d_dst;
    int64_t *d_soff, *d_sbytes, *d_poff, *d_pbytes;
    int32_t *d_psrc, *d_psig, *d_pwait, *d_sdst;
    const void** h_src = slot.Alloc<const void*>(ns + 1, &d_src);
    void** h_self = slot.Alloc<void*>(ns + 1, &d_self);
    int64_t* h_soff = slot.Alloc<int64_t>(ns + 1, &d_soff);
    int64_t* h_sbytes = slot.Alloc<int64_t>(ns + 1, &d_sbytes);
    int32_t* h_sdst = slot.Alloc<int32_t>(ns + 1, &d_sdst);
    void** h_dst = slot.Alloc<void*>(np + 1, &d_dst);
    int64_t* h_poff = slot.Alloc<int64_t>(np + 1, &d_poff);
    int64_t* h_pbytes = slot.Alloc<int64_t>(np + 1, &d_pbytes);
    int32_t* h_psrc = slot.Alloc<int32_t>(np + 1, &d_psrc);
    int32_t* h_psig = slot.Alloc<int32_t>(np + 1, &d_psig);
    int32_t* h_pwait = slot.Alloc<int32_t>(np + 1, &d_pwait);
    if (!h_src || !h_self || !h_soff || !h_sbytes || !h_dst || !h_poff || !h_pbytes ||
        !h_psrc || !h_psig || !h_pwait || !h_sdst)
      throw std::runtime_error("exchange plan does not fit a descriptor slot");
    for (size_t i = 0; i < ns; ++i) {
      h_src[i] = stage[i].src;
      h_self[i] = stage[i].self_dst;
      h_soff[i] = stage[i].off;
      h_sbytes[i] = stage[i].bytes;
      h_sdst[i] = stage[i].dst;
    }
    for (size_t i = 0; i < np; ++i) {
      h_dst[i] = pull[i].dst;
      h_poff[i] = pull[i].off;
      h_pbytes[i] = pull[i].bytes;
      h_psrc[i] = pull[i].src_rank;
      h_psig[i] = pull[i].sig_rank;
      h_pwait[i] = static_cast<int32_t>(before[pull[i].block]);
    }
    ring_.Commit(slot, stream_);
    plan.n_stage = static_cast<int>(ns);
    plan.st_src = d_src;
    plan.st_self = d_self;
    plan.st_off = d_soff;
    plan.st_bytes = d_sbytes;
    plan.st_dst = d_sdst;
    plan.n_pull = static_cast<int>(np);
    plan.pl_dst = d_dst;
    plan.pl_off = d_poff;
    plan.pl_bytes = d_pbytes;
    plan.pl_src = d_psrc;
    plan.pl_sig = d_psig;
    plan.pl_wait = d_pwait;
    kern::SymmCtx ctx = MakeCtx(set, sync.done_epochs, region_off);
    host_trace::Mark("plan (ring)");
    err = kern::LaunchExchange(plan, sync, ctas, ctx, stream_);
    host_trace::Mark("launch");
    ring_.Release(slot, stream_);
  }
  if (err != cudaSuccess)
    throw std::runtime_error(std::string("exchange kernel launch failed: ") +
                             cudaGetErrorString(err));
}

namespace {
int64_t ExchangeRegionBytes(const SymmSet& set) {
  return set.xchg_bytes > 0 ? set.xchg_bytes : static_cast<int64_t>(set.data_bytes);
}
}  // namespace

bool GpuOps::ExchangePushes(const SymmSet& set, int64_t total_bytes) const {
  // Writing into other ranks' regions is only safe for the credit-guarded
  // regions of the global set: nothing else ever touches those. Measured on
  // B200: with two ranks pulling wins above about 1 MB (one NVLink pass, no
  // second local pass); from three ranks on, stores into the receivers'
  // regions beat loads from several peers at every size (4 ranks, 256 MB
  // allgather: 468 us pushed, 599 us pulled).
  if (set.world <= 1 || set.xchg_bytes <= 0) return false;
  if (exchange_push_max_ >= 0 && total_bytes <= exchange_push_max_) return true;
  return set.world >= 3 && exchange_push_max_ != 0;
}

bool GpuOps::ExchangeUsesCopyEngine(const SymmSet& set, int64_t total_bytes, int64_t smallest,
                                    size_t remote_blocks, bool allgather) const {
  // A copy-engine peer copy reaches 750-765 GB/s per direction on B200;
  // SM-driven NVLink traffic (this kernel and NCCL alike) 430-530 GB/s. But
  // staging, barrier and copies run one after the other, so the copy engines
  // only win where the kernel is furthest from the link rate: measured at 4
  // ranks, allgather 256 MB 385 us (kernel 463, NCCL path 394), 1 GB 1358 us
  // (1851, 1413); at 64 MB and for every alltoall size the kernel is faster,
  // and at 2 ranks the two tie. HOROVOD_EXCHANGE_COPY_ENGINE_MIN_BYTES
  // overrides for all exchange ops (0 = never).
  if (set.world <= 1 || set.xchg_bytes <= 0 || smallest < (256 << 10) || remote_blocks > 256)
    return false;
  if (exchange_ce_min_ >= 0) return exchange_ce_min_ > 0 && total_bytes >= exchange_ce_min_;
  return allgather && set.world >= 3 && total_bytes >= (int64_t(128) << 20);
}

namespace {
// Totals over the blocks that cross NVLink (the same on every rank).
struct RemoteStats { int64_t total = 0, smallest = 0; size_t count = 0; };
RemoteStats RemoteBlockStats(const std::vector<ExchangeBlock>& blocks, int world) {
  RemoteStats st;
  for (auto& b : blocks) {
    st.total += b.bytes;
    const bool remote = world > 1 && (b.dst_rank < 0 || b.dst_rank != b.src_rank);
    if (!remote || b.bytes == 0) continue;
    st.smallest = st.count == 0 ? b.bytes : std::min(st.smallest, b.bytes);
    ++st.count;
  }
  return st;
}
}  // namespace

Status GpuOps::SymmBroadcast(std::vector<TensorTableEntry>& entries,
                             SymmSet& set) {
  Timeline& tl = state_.timeline;
  WaitForInputs(entries);
  host_trace::Mark("inputs");
  ActStart(entries, HVD_ACT_FUSED_KERNEL);
  std::vector<ExchangeBlock> blocks;
  for (auto& e : entries) {
    ExchangeBlock b;
    b.src_rank = e.root_rank;
    b.dst_rank = -1;
    b.src = static_cast<const char*>(e.input);
    b.dst = static_cast<char*>(e.output);
    // The root already holds the data unless it asked for a separate output.
    if (set.rank == e.root_rank && e.input == e.output) b.dst = nullptr;
    b.bytes = e.size_bytes();
    blocks.push_back(b);
  }
  // From three ranks on the root writes everybody's region at once through
  // the multicast mapping (its NVLink egress is S instead of (N-1) S) and the
  // receivers copy out of their own region; with two ranks the peer pulls
  // large messages. (Only with the credit-guarded regions: nobody else ever
  // writes those.)
  const RemoteStats rs = RemoteBlockStats(blocks, set.world);
  const bool push = ExchangePushes(set, rs.total) ||
                    (set.mc != nullptr && set.world >= 3 && set.xchg_bytes > 0);
  // (A pulled broadcast would cost the root N-1 times the message on its
  // NVLink egress, so the copy engines only serve the two-rank case.)
  const bool ce = !push && ExchangeUsesCopyEngine(set, rs.total, rs.smallest, rs.count, false);
  PlanExchangeRounds(blocks, set.rank, set.world, ExchangeRegionBytes(set), push,
            [&](const std::vector<StageSeg>& o, const std::vector<PullSeg>& i,
                int64_t round_bytes, const std::vector<RoundBlock>& round) {
              LaunchExchangeSegments(o, i, set, round_bytes, round, ce);
            });
  ActEnd(entries);
  return Complete(entries);
}

Status GpuOps::SymmAllgather(std::vector<TensorTableEntry>& entries,
                             const Response& response, SymmSet& set) {
  Timeline& tl = state_.timeline;
  const int n = set.world;
  WaitForInputs(entries);
  host_trace::Mark("inputs");
  std::vector<ExchangeBlock> blocks;
  for (size_t i = 0; i < entries.size(); ++i) {
    TensorTableEntry& e = entries[i];
    int64_t slice = static_cast<int64_t>(DataTypeSize(e.dtype));
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    int64_t rows = 0;
    for (int r = 0; r < n; ++r) rows += response.tensor_sizes[i * n + r];
    std::vector<int64_t> dims = e.shape.to_vector();
    dims[0] = rows;
    tl.ActivityStart(e.name, HVD_ACT_ALLOCATE_OUTPUT);
    void* out = nullptr;
    Status st = e.context->AllocateOutput(TensorShape(dims), stream_, &out);
    tl.ActivityEnd(e.name);
    if (!st.ok()) return st;
    e.output = out;
    int64_t disp = 0;
    for (int r = 0; r < n; ++r) {
      ExchangeBlock b;
      b.src_rank = r;
      b.dst_rank = -1;
      b.src = r == set.rank ? static_cast<const char*>(e.input) : nullptr;
      b.dst = static_cast<char*>(out) + disp;
      b.bytes = response.tensor_sizes[i * n + r] * slice;
      disp += b.bytes;
      blocks.push_back(b);
    }
  }
  host_trace::Mark("outputs");
  ActStart(entries, HVD_ACT_FUSED_KERNEL);
  const RemoteStats rs = RemoteBlockStats(blocks, set.world);
  const bool ce = ExchangeUsesCopyEngine(set, rs.total, rs.smallest, rs.count, true);
  PlanExchangeRounds(blocks, set.rank, set.world, ExchangeRegionBytes(set),
                     !ce && ExchangePushes(set, rs.total),
            [&](const std::vector<StageSeg>& o, const std::vector<PullSeg>& i,
                int64_t round_bytes, const std::vector<RoundBlock>& round) {
              LaunchExchangeSegments(o, i, set, round_bytes, round, ce);
            });
  ActEnd(entries);
  return Complete(entries);
}

Status GpuOps::SymmAlltoall(std::vector<TensorTableEntry>& entries, const Response& response,
                            ProcessSet& ps, SymmSet& set) {
  Timeline& tl = state_.timeline;
  const int n = set.world, me = set.rank;
  WaitForInputs(entries);
  std::vector<ExchangeBlock> blocks;
  for (auto& e : entries) {
    int64_t slice = static_cast<int64_t>(DataTypeSize(e.dtype));
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    // Full split matrix over the control plane: all[r * n + p] = rows rank r
    // sends to rank p.
    std::vector<int32_t> all(static_cast<size_t>(n) * n);
    host_trace::Mark("inputs");
    std::vector<int32_t> even;
    if (AlltoallEvenRows(response, n, &even)) {
      // Every rank asked for an even split and the response carries every
      // rank's first dimension: the table is known without an exchange.
      for (int r = 0; r < n; ++r)
        for (int p = 0; p < n; ++p) all[r * n + p] = even[r];
    } else {
      ps.comm.Allgather(e.splits.data(), sizeof(int32_t) * n, all.data());
    }
    host_trace::Mark("splits");
    std::vector<int32_t> recv(n);
    int64_t rows = 0;
    for (int r = 0; r < n; ++r) {
      recv[r] = all[r * n + me];
      rows += recv[r];
    }
    std::vector<int64_t> dims = e.shape.to_vector();
    dims[0] = rows;
    tl.ActivityStart(e.name, HVD_ACT_ALLOCATE_OUTPUT);
    void* out = nullptr;
    Status st = e.context->AllocateOutput(TensorShape(dims), stream_, &out);
    tl.ActivityEnd(e.name);
    if (!st.ok()) return st;
    e.output = out;
    e.context->SetReceivedSplits(recv);
    std::vector<int64_t> send_off(n, 0), recv_off(n, 0);
    for (int p = 1; p < n; ++p) {
      send_off[p] = send_off[p - 1] + e.splits[p - 1] * slice;
      recv_off[p] = recv_off[p - 1] + recv[p - 1] * slice;
    }
    for (int r = 0; r < n; ++r) {
      // Rank r sends to r+1, r+2, ... in turn: at any time every GPU is the
      // target of one sender instead of everybody writing to rank 0 first.
      for (int j = 1; j <= n; ++j) {
        const int p = (r + j) % n;
        ExchangeBlock b;
        b.src_rank = r;
        b.dst_rank = p;
        b.bytes = static_cast<int64_t>(all[r * n + p]) * slice;
        b.src = r == me ? static_cast<const char*>(e.input) + send_off[p] : nullptr;
        b.dst = p == me ? static_cast<char*>(out) + recv_off[r] : nullptr;
        blocks.push_back(b);
      }
    }
  }
  ActStart(entries, HVD_ACT_FUSED_KERNEL);
  const RemoteStats rs = RemoteBlockStats(blocks, set.world);
  const bool ce = ExchangeUsesCopyEngine(set, rs.total, rs.smallest, rs.count, false);
  PlanExchangeRounds(blocks, set.rank, set.world, ExchangeRegionBytes(set),
                     !ce && ExchangePushes(set, rs.total),
            [&](const std::vector<StageSeg>& o, const std::vector<PullSeg>& i,
                int64_t round_bytes, const std::vector<RoundBlock>& round) {
              LaunchExchangeSegments(o, i, set, round_bytes, round, ce);
            });
  ActEnd(entries);
  return Complete(entries);
}

}  // namespace hvd
