// Broadcast, allgather and alltoall on device tensors, all expressed as
// segment lists for the exchange kernel: outbound segments go from local
// tensors into the staging buffer of their destination rank(s), inbound
// segments go from the local staging buffer into the final tensors.
#include <algorithm>
#include <cstring>

#include "../common/logging.h"
#include "../common/process_set.h"
#include "gpu_internal.h"

namespace hvd {

namespace {
constexpr int64_t STAGING_ALIGN = 256;
}

void GpuOps::LaunchExchangeSegments(const std::vector<OutSeg>& out,
                                    const std::vector<InSeg>& in, SymmSet& set,
                                    int64_t round_bytes,
                                    const std::vector<RoundBlock>& round) {
  if (exchange_pipeline_ && set.world > 1 && round_bytes >= (8 << 20) &&
      LaunchExchangePipelined(out, in, set, round_bytes, round))
    return;
  const size_t no = out.size(), ni = in.size();
  // The grid size must be the same on every rank (CTA b meets CTA b of its
  // peers), so it is derived from the bytes of the whole round, which all
  // ranks know, not from this rank's share of them.
  const int64_t bytes = round_bytes;
  kern::ExchangePlan plan;
  std::memset(&plan, 0, sizeof(plan));
  cudaError_t err;
  if (no <= kern::INLINE_SEGMENTS && ni <= kern::INLINE_SEGMENTS) {
    // Short plan: carried in the kernel parameters.
    kern::InlineExchange inl;
    inl.n_out = static_cast<int>(no);
    inl.n_in = static_cast<int>(ni);
    for (size_t i = 0; i < no; ++i) {
      inl.out_src[i] = out[i].src;
      inl.out_staging_off[i] = out[i].staging_off;
      inl.out_bytes[i] = out[i].bytes;
      inl.out_dst_rank[i] = out[i].dst;
    }
    for (size_t i = 0; i < ni; ++i) {
      inl.in_dst[i] = in[i].dst;
      inl.in_staging_off[i] = in[i].staging_off;
      inl.in_bytes[i] = in[i].bytes;
    }
    if (no == 0 && ni == 0) inl.n_out = 0;
    kern::SymmCtx ctx = MakeCtx(set, kern::EPOCHS_PER_LAUNCH);
    // An empty inline plan would read as "not used": give the kernel the
    // (equally empty) device plan in that case.
    err = kern::LaunchExchange(plan, PickCtas(bytes), ctx, stream_,
                               (no || ni) ? &inl : nullptr);
  } else {
    DescriptorRing::Slot slot = ring_.Acquire();
    const void** d_src;
    int64_t *d_ooff, *d_obytes, *d_ioff, *d_ibytes;
    int32_t* d_dst_rank;
    void** d_dst;
    const void** h_src = slot.Alloc<const void*>(no + 1, &d_src);
    int64_t* h_ooff = slot.Alloc<int64_t>(no + 1, &d_ooff);
    int64_t* h_obytes = slot.Alloc<int64_t>(no + 1, &d_obytes);
    int32_t* h_dst_rank = slot.Alloc<int32_t>(no + 1, &d_dst_rank);
    void** h_dst = slot.Alloc<void*>(ni + 1, &d_dst);
    int64_t* h_ioff = slot.Alloc<int64_t>(ni + 1, &d_ioff);
    int64_t* h_ibytes = slot.Alloc<int64_t>(ni + 1, &d_ibytes);
    if (!h_src || !h_ooff || !h_obytes || !h_dst_rank || !h_dst || !h_ioff || !h_ibytes)
      throw std::runtime_error("exchange plan does not fit a descriptor slot");
    for (size_t i = 0; i < no; ++i) {
      h_src[i] = out[i].src;
      h_ooff[i] = out[i].staging_off;
      h_obytes[i] = out[i].bytes;
      h_dst_rank[i] = out[i].dst;
    }
    for (size_t i = 0; i < ni; ++i) {
      h_dst[i] = in[i].dst;
      h_ioff[i] = in[i].staging_off;
      h_ibytes[i] = in[i].bytes;
    }
    ring_.Commit(slot, stream_);
    plan.n_out = static_cast<int>(no);
    plan.out_src = d_src;
    plan.out_staging_off = d_ooff;
    plan.out_bytes = d_obytes;
    plan.out_dst_rank = d_dst_rank;
    plan.n_in = static_cast<int>(ni);
    plan.in_dst = d_dst;
    plan.in_staging_off = d_ioff;
    plan.in_bytes = d_ibytes;
    kern::SymmCtx ctx = MakeCtx(set, kern::EPOCHS_PER_LAUNCH);
    err = kern::LaunchExchange(plan, PickCtas(bytes), ctx, stream_);
    ring_.Release(slot, stream_);
  }
  if (err != cudaSuccess)
    throw std::runtime_error(std::string("exchange kernel launch failed: ") +
                             cudaGetErrorString(err));
}

// Plan for the pipelined kernel. Every rank derives the same numbers from the
// round's block list: the grid size, the chunks per block, how many chunks a
// source has published before each of its blocks, and the epochs the launch
// consumes (the largest chunk total of any rank, plus one for the final barrier).
// Returns false (nothing launched) when the plan does not fit a descriptor slot.
bool GpuOps::LaunchExchangePipelined(const std::vector<OutSeg>& out,
                                     const std::vector<InSeg>& in, SymmSet& set,
                                     int64_t round_bytes,
                                     const std::vector<RoundBlock>& round) {
  const size_t no = out.size(), ni = in.size();
  const int ctas = PickCtas(round_bytes);
  const int64_t chunk = exchange_chunk_bytes_ / 256 * 256;
  std::vector<int64_t> published(set.world, 0);   // chunks per source so far
  std::vector<int64_t> before(round.size(), 0);   // ... before each block
  for (size_t i = 0; i < round.size(); ++i) {
    const int src = round[i].src_rank;
    if (src < 0 || src >= set.world) return false;
    before[i] = published[src];
    published[src] += kern::ExchangeChunkCount(round[i].bytes, ctas, chunk);
  }
  const int64_t most = *std::max_element(published.begin(), published.end());
  if (most + 1 > (int64_t(1) << 30)) return false;

  DescriptorRing::Slot slot = ring_.Acquire();
  const void** d_src;
  int64_t *d_ooff, *d_obytes, *d_ioff, *d_ibytes;
  int32_t *d_dst_rank, *d_isrc, *d_iwait;
  void** d_dst;
  const void** h_src = slot.Alloc<const void*>(no + 1, &d_src);
  int64_t* h_ooff = slot.Alloc<int64_t>(no + 1, &d_ooff);
  int64_t* h_obytes = slot.Alloc<int64_t>(no + 1, &d_obytes);
  int32_t* h_dst_rank = slot.Alloc<int32_t>(no + 1, &d_dst_rank);
  void** h_dst = slot.Alloc<void*>(ni + 1, &d_dst);
  int64_t* h_ioff = slot.Alloc<int64_t>(ni + 1, &d_ioff);
  int64_t* h_ibytes = slot.Alloc<int64_t>(ni + 1, &d_ibytes);
  int32_t* h_isrc = slot.Alloc<int32_t>(ni + 1, &d_isrc);
  int32_t* h_iwait = slot.Alloc<int32_t>(ni + 1, &d_iwait);
  if (!h_src || !h_ooff || !h_obytes || !h_dst_rank || !h_dst || !h_ioff || !h_ibytes ||
      !h_isrc || !h_iwait) {
    // Nothing was copied or launched: hand the slot back unused.
    ring_.Release(slot, stream_);
    return false;
  }
  for (size_t i = 0; i < no; ++i) {
    h_src[i] = out[i].src;
    h_ooff[i] = out[i].staging_off;
    h_obytes[i] = out[i].bytes;
    h_dst_rank[i] = out[i].dst;
  }
  for (size_t i = 0; i < ni; ++i) {
    h_dst[i] = in[i].dst;
    h_ioff[i] = in[i].staging_off;
    h_ibytes[i] = in[i].bytes;
    h_isrc[i] = in[i].src_rank;
    h_iwait[i] = static_cast<int32_t>(before[in[i].block]);
  }
  ring_.Commit(slot, stream_);
  kern::PipelinePlan plan;
  std::memset(&plan, 0, sizeof(plan));
  plan.n_out = static_cast<int>(no);
  plan.out_src = d_src;
  plan.out_staging_off = d_ooff;
  plan.out_bytes = d_obytes;
  plan.out_dst_rank = d_dst_rank;
  plan.n_in = static_cast<int>(ni);
  plan.in_dst = d_dst;
  plan.in_staging_off = d_ioff;
  plan.in_bytes = d_ibytes;
  plan.in_src_rank = d_isrc;
  plan.in_wait_base = d_iwait;
  plan.chunk_bytes = chunk;
  plan.done_epochs = static_cast<uint32_t>(most + 1);
  kern::SymmCtx ctx = MakeCtx(set, plan.done_epochs);
  cudaError_t err = kern::LaunchExchangePipelined(plan, ctas, ctx, stream_);
  ring_.Release(slot, stream_);
  if (err != cudaSuccess)
    throw std::runtime_error(std::string("pipelined exchange launch failed: ") +
                             cudaGetErrorString(err));
  return true;
}

// Every rank builds the same global list of "blocks" (source rank, bytes,
// who receives it); blocks are laid out in the staging buffer in order and
// processed in rounds that fit its capacity. A block larger than the
// capacity is cut into parts first. All of this is deterministic, so the
// ranks agree on rounds and offsets without talking.
namespace {
struct Block {
  int src_rank;        // set rank that owns the data
  int dst_rank;        // receiving set rank, or -1 for everybody
  const char* src;     // valid on src_rank only
  char* dst;           // where this rank wants the data (null = not wanted)
  int64_t bytes;
};
}  // namespace

static void RunBlocks(GpuOps* self, std::vector<Block>& blocks, SymmSet& set,
                      const std::function<void(const std::vector<GpuOps::OutSeg>&,
                                               const std::vector<GpuOps::InSeg>&,
                                               int64_t,
                                               const std::vector<GpuOps::RoundBlock>&)>& launch) {
  (void)self;
  const int64_t cap = static_cast<int64_t>(set.data_bytes);
  // Split oversized blocks.
  std::vector<Block> parts;
  for (auto& b : blocks) {
    int64_t pos = 0;
    if (b.bytes == 0) continue;
    while (pos < b.bytes) {
      int64_t take = std::min(b.bytes - pos, cap / 2 / STAGING_ALIGN * STAGING_ALIGN);
      Block p = b;
      p.src = b.src ? b.src + pos : nullptr;
      p.dst = b.dst ? b.dst + pos : nullptr;
      p.bytes = take;
      parts.push_back(p);
      pos += take;
    }
  }
  size_t next = 0;
  while (next < parts.size()) {
    std::vector<GpuOps::OutSeg> out;
    std::vector<GpuOps::InSeg> in;
    // Offsets are per destination buffer: a block for everybody advances all
    // cursors, a point-to-point block only its destination's.
    std::vector<int64_t> cursor(set.world, 0);
    size_t n = 0;
    int64_t round_bytes = 0;
    std::vector<GpuOps::RoundBlock> round;
    while (next + n < parts.size() && n < 4096) {
      const Block& b = parts[next + n];
      int64_t padded = RoundUp(b.bytes, STAGING_ALIGN);
      int64_t off;
      if (b.dst_rank < 0) {
        off = *std::max_element(cursor.begin(), cursor.end());
        if (off + padded > cap) break;
        for (auto& c : cursor) c = off + padded;
      } else {
        off = cursor[b.dst_rank];
        if (off + padded > cap) break;
        cursor[b.dst_rank] = off + padded;
      }
      if (b.src_rank == set.rank)
        out.push_back({b.src, off, b.bytes, b.dst_rank});
      if ((b.dst_rank < 0 || b.dst_rank == set.rank) && b.dst != nullptr)
        in.push_back({b.dst, off, b.bytes, b.src_rank, static_cast<int32_t>(round.size())});
      round.push_back({b.src_rank, b.bytes});
      round_bytes += b.bytes;
      ++n;
    }
    if (n == 0) throw std::runtime_error("exchange block exceeds staging capacity");
    launch(out, in, round_bytes, round);
    next += n;
  }
}

Status GpuOps::SymmBroadcast(std::vector<TensorTableEntry>& entries,
                             SymmSet& set) {
  Timeline& tl = state_.timeline;
  WaitForInputs(entries);
  tl.ActivityStartAll(entries, HVD_ACT_FUSED_KERNEL);
  std::vector<Block> blocks;
  for (auto& e : entries) {
    Block b;
    b.src_rank = e.root_rank;
    b.dst_rank = -1;
    b.src = static_cast<const char*>(e.input);
    b.dst = static_cast<char*>(e.output);
    // The root already holds the data unless it asked for a separate output.
    if (set.rank == e.root_rank && e.input == e.output) b.dst = nullptr;
    b.bytes = e.size_bytes();
    blocks.push_back(b);
  }
  RunBlocks(this, blocks, set,
            [&](const std::vector<OutSeg>& o, const std::vector<InSeg>& i, int64_t round_bytes,
                const std::vector<RoundBlock>& round) {
              LaunchExchangeSegments(o, i, set, round_bytes, round);
            });
  tl.ActivityEndAll(entries);
  return Complete(entries);
}

Status GpuOps::SymmAllgather(std::vector<TensorTableEntry>& entries,
                             const Response& response, SymmSet& set) {
  Timeline& tl = state_.timeline;
  const int n = set.world;
  WaitForInputs(entries);
  std::vector<Block> blocks;
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
      Block b;
      b.src_rank = r;
      b.dst_rank = -1;
      b.src = r == set.rank ? static_cast<const char*>(e.input) : nullptr;
      b.dst = static_cast<char*>(out) + disp;
      b.bytes = response.tensor_sizes[i * n + r] * slice;
      disp += b.bytes;
      blocks.push_back(b);
    }
  }
  tl.ActivityStartAll(entries, HVD_ACT_FUSED_KERNEL);
  RunBlocks(this, blocks, set,
            [&](const std::vector<OutSeg>& o, const std::vector<InSeg>& i, int64_t round_bytes,
                const std::vector<RoundBlock>& round) {
              LaunchExchangeSegments(o, i, set, round_bytes, round);
            });
  tl.ActivityEndAll(entries);
  return Complete(entries);
}

Status GpuOps::SymmAlltoall(std::vector<TensorTableEntry>& entries,
                            ProcessSet& ps, SymmSet& set) {
  Timeline& tl = state_.timeline;
  const int n = set.world, me = set.rank;
  WaitForInputs(entries);
  std::vector<Block> blocks;
  for (auto& e : entries) {
    int64_t slice = static_cast<int64_t>(DataTypeSize(e.dtype));
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    // Full split matrix over the control plane: all[r * n + p] = rows rank r
    // sends to rank p.
    std::vector<int32_t> all(static_cast<size_t>(n) * n);
    ps.comm.Allgather(e.splits.data(), sizeof(int32_t) * n, all.data());
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
        Block b;
        b.src_rank = r;
        b.dst_rank = p;
        b.bytes = static_cast<int64_t>(all[r * n + p]) * slice;
        b.src = r == me ? static_cast<const char*>(e.input) + send_off[p] : nullptr;
        b.dst = p == me ? static_cast<char*>(out) + recv_off[r] : nullptr;
        blocks.push_back(b);
      }
    }
  }
  tl.ActivityStartAll(entries, HVD_ACT_FUSED_KERNEL);
  RunBlocks(this, blocks, set,
            [&](const std::vector<OutSeg>& o, const std::vector<InSeg>& i, int64_t round_bytes,
                const std::vector<RoundBlock>& round) {
              LaunchExchangeSegments(o, i, set, round_bytes, round);
            });
  tl.ActivityEndAll(entries);
  return Complete(entries);
}

}  // namespace hvd
