// Device collectives over symmetric memory: builds the per-launch
// descriptors, picks algorithm and grid, and launches the NVLink kernels on
// the communication stream.
#include <algorithm>
#include <cstring>

#include "../common/logging.h"
#include "../common/process_set.h"
#include "gpu_internal.h"
#include "host_trace.h"

namespace hvd {

namespace {

// A run of elements of one tensor that goes into one launch. Tensors larger
// than the staging buffer are cut into several pieces.
struct Piece {
  const char* in;
  char* out;
  int64_t count;
};

constexpr int64_t STAGING_ALIGN = 256;

}  // namespace

Status GpuOps::SymmAllreduce(std::vector<TensorTableEntry>& entries,
                             const Response& response, SymmSet& set,
                             bool adasum) {
  Timeline& tl = state_.timeline;
  const DataType dtype = response.dtype;
  // Adasum stages fp32 whatever the tensor type.
  const DataType wire = (adasum && set.world > 1)
                            ? DataType::FLOAT32
                            : (adasum ? dtype : response.wire_dtype);
  const int64_t es = static_cast<int64_t>(DataTypeSize(dtype));
  const int64_t ws = static_cast<int64_t>(DataTypeSize(wire));
  const int64_t align_elems = FUSION_ALIGN_BYTES / ws;

  WaitForInputs(entries);
  // A group of one that reduces in place with unit scale changes nothing:
  // no kernel at all (what a single-GPU run of a data-parallel script does
  // for every gradient).
  if (set.world == 1 && !adasum && wire == dtype &&
      response.prescale * response.postscale == 1.0) {
    bool in_place = true;
    for (auto& e : entries)
      if (e.input != e.output) in_place = false;
    if (in_place) return Complete(entries);
  }
  ActStart(entries, HVD_ACT_FUSED_KERNEL);
  // (A response with fewer devices than ranks means somebody has joined and
  // contributes zeros: everybody stages in that case.)
  if (!adasum && set.world > 1 && wire == dtype &&
      static_cast<int>(response.devices.size()) == set.world) {
    Status st;
    if (TryInplaceAllreduce(entries, response, set, &st)) {
      if (!st.ok()) return st;
      ActEnd(entries);
      return Complete(entries);
    }
  }

  // Room for data; Adasum also keeps 3 doubles per tensor per level behind it.
  int64_t capacity = static_cast<int64_t>(set.data_bytes);
  if (adasum) capacity -= RoundUp(int64_t(entries.size()) * 3 * 8 * 4 + 4096, 4096);
  const int64_t cap_elems = capacity / ws / align_elems * align_elems;

  // Cut into pieces no larger than the staging capacity.
  std::vector<Piece> pieces;
  for (auto& e : entries) {
    int64_t n = e.num_elements(), pos = 0;
    if (n == 0) continue;
    if (adasum && n > cap_elems)
      return Status::InvalidArgument(
          "Adasum tensor '" + e.name + "' does not fit the symmetric staging "
          "buffer; raise HOROVOD_SYMM_BUFFER_MB.");
    while (pos < n) {
      int64_t take = std::min(n - pos, cap_elems);
      Piece p;
      p.in = e.input ? static_cast<const char*>(e.input) + pos * es : nullptr;
      p.out = e.output ? static_cast<char*>(e.output) + pos * es : nullptr;
      p.count = take;
      pieces.push_back(p);
      pos += take;
    }
  }

  size_t next = 0;
  while (next < pieces.size()) {
    // Greedy batch of pieces that fits the staging buffer and one
    // descriptor slot.
    const size_t max_n = std::min<size_t>(pieces.size() - next,
                                          (ring_.slot_bytes() - 4096) / 40);
    int64_t total = 0;
    size_t n = 0;
    while (n < max_n) {
      int64_t padded = RoundUp(pieces[next + n].count, align_elems);
      if (n > 0 && total + padded > cap_elems) break;
      total += padded;
      ++n;
    }
    // Short lists ride in the kernel parameters; long ones go through the
    // descriptor ring (one small host-to-device copy).
    const bool use_inline = inline_descriptors_ &&
                            n <= static_cast<size_t>(kern::INLINE_TENSORS);
    kern::InlineTensors inl;
    inl.n = 0;
    kern::TensorList list = {static_cast<int>(n), nullptr, nullptr, nullptr, nullptr};
    DescriptorRing::Slot slot;
    int64_t *h_off, *h_cnt;
    const void** h_in;
    void** h_out;
    if (use_inline) {
      inl.n = static_cast<int>(n);
      h_off = inl.offsets;
      h_cnt = inl.counts;
      h_in = inl.in;
      h_out = inl.out;
    } else {
      slot = ring_.Acquire();
      int64_t *d_off, *d_cnt;
      const void** d_in;
      void** d_out;
      h_off = slot.Alloc<int64_t>(n + 1, &d_off);
      h_cnt = slot.Alloc<int64_t>(n, &d_cnt);
      h_in = slot.Alloc<const void*>(n, &d_in);
      h_out = slot.Alloc<void*>(n, &d_out);
      if (!h_off || !h_cnt || !h_in || !h_out)
        return Status::UnknownError("descriptor slot too small");
      list.offsets = d_off;
      list.counts = d_cnt;
      list.in = d_in;
      list.out = d_out;
    }
    int64_t off = 0;
    for (size_t i = 0; i < n; ++i) {
      const Piece& p = pieces[next + i];
      h_off[i] = off;
      h_cnt[i] = p.count;
      h_in[i] = p.in;
      h_out[i] = p.out;
      off += RoundUp(p.count, align_elems);
    }
    h_off[n] = off;
    if (!use_inline) ring_.Commit(slot, stream_);

    const int64_t bytes = off * ws;
    cudaError_t err;
    if (adasum && set.world > 1) {
      if (use_inline) {
        // The Adasum kernels read the list from device memory.
        slot = ring_.Acquire();
        int64_t *d_off, *d_cnt;
        const void** d_in;
        void** d_out;
        int64_t* o = slot.Alloc<int64_t>(n + 1, &d_off);
        int64_t* c = slot.Alloc<int64_t>(n, &d_cnt);
        const void** ip = slot.Alloc<const void*>(n, &d_in);
        void** op = slot.Alloc<void*>(n, &d_out);
        std::memcpy(o, h_off, (n + 1) * sizeof(int64_t));
        std::memcpy(c, h_cnt, n * sizeof(int64_t));
        std::memcpy(ip, h_in, n * sizeof(void*));
        std::memcpy(op, h_out, n * sizeof(void*));
        list.offsets = d_off;
        list.counts = d_cnt;
        list.in = d_in;
        list.out = d_out;
        ring_.Commit(slot, stream_);
      }
      kern::SymmCtx ctx = MakeCtx(set, kern::ADASUM_EPOCHS);
      int64_t scratch_off = RoundUp(bytes, 4096);
      // Room behind the scratch for a local copy of the partner's half, if
      // the staging area has it.
      const int64_t scratch_bytes = RoundUp(int64_t(n) * 3 * 8 * 4 + 4096, 4096);
      int64_t copy_off = scratch_off + scratch_bytes;
      if (copy_off + bytes / 2 + 4096 > static_cast<int64_t>(set.data_bytes)) copy_off = -1;
      err = kern::LaunchAdasum(list, dtype, response.prescale,
                               response.postscale, scratch_off, PickCtas(bytes),
                               ctx, stream_, copy_off);
      ring_.Release(slot, stream_);
    } else {
      kern::Algo algo = PickAlgo(set, wire, bytes);
      int ctas = PickCtas(bytes);
      // A single rank waits for nobody: use the whole GPU for the copy.
      if (algo == kern::Algo::LOCAL && forced_ctas_ <= 0)
        ctas = static_cast<int>(std::min<int64_t>(296, std::max<int64_t>(1, bytes >> 16)));
      int64_t staging_off = 0;
      bool skip_end = false;
      if (algo == kern::Algo::ONESHOT && set.oneshot_bytes >= bytes) {
        staging_off = set.oneshot_off[set.oneshot_count++ & 1];
        skip_end = true;
      }
      // Two-shot / NVLS launches of 8 MB and more run as a pipeline over
      // sub-chunks (pack, reduce and unpack of neighbouring sub-chunks
      // overlap); every rank derives the same step count from the same sizes.
      int64_t sub_vecs = 0;
      uint32_t epochs = kern::EPOCHS_PER_LAUNCH;
      if (algo == kern::Algo::TWOSHOT || algo == kern::Algo::NVLS) {
        if (bytes >= allreduce_pipeline_min_ && allreduce_subchunk_bytes_ > 0)
          sub_vecs = allreduce_subchunk_bytes_ / 16;
        epochs = std::max(epochs, kern::FusedAllreduceEpochs(bytes / 16, set.world, ctas, sub_vecs));
      }
      kern::SymmCtx ctx = MakeCtx(set, epochs, staging_off, skip_end);
      ctx.sub_chunk_vecs = sub_vecs;
      host_trace::Mark("plan");
      err = kern::LaunchFusedAllreduce(list, dtype, adasum ? dtype : wire,
                                       response.prescale, response.postscale,
                                       algo, ctas, ctx, stream_,
                                       use_inline ? &inl : nullptr);
      host_trace::Mark("launch");
      if (!use_inline) ring_.Release(slot, stream_);
    }
    if (err != cudaSuccess)
      return Status::UnknownError(std::string("fused allreduce launch failed: ") +
                                  cudaGetErrorString(err));
    next += n;
  }
  ActEnd(entries);
  return Complete(entries);
}

bool GpuOps::TryInplaceAllreduce(std::vector<TensorTableEntry>& entries,
                                 const Response& response, SymmSet& set,
                                 Status* status) {
  const DataType dtype = response.dtype;
  if (dtype != DataType::FLOAT32 && dtype != DataType::FLOAT16 &&
      dtype != DataType::BFLOAT16 && dtype != DataType::FLOAT64)
    return false;
  const int64_t es = static_cast<int64_t>(DataTypeSize(dtype));
  struct R { int64_t off, bytes; };
  std::vector<R> ranges;
  for (auto& e : entries) {
    if (e.input == nullptr || e.input != e.output) return false;  // also joined ranks
    int64_t off = 0, bytes = e.num_elements() * es;
    if (bytes == 0) continue;
    if (!InSymmHeap(e.input, bytes, &off) || (off & 15) != 0) return false;
    ranges.push_back({off, bytes});
  }
  // Every rank must take the same decision: tensors are symmetric by
  // construction (same allocation sequence), so offsets agree; a rank whose
  // tensor is elsewhere has a different layout on all ranks alike.
  if (ranges.empty()) return false;
  std::sort(ranges.begin(), ranges.end(), [](const R& a, const R& b) { return a.off < b.off; });
  std::vector<R> merged;
  for (auto& r : ranges) {
    // Merge neighbours; a range with a ragged tail cannot be extended.
    if (!merged.empty() && merged.back().off + merged.back().bytes == r.off &&
        (merged.back().bytes & 15) == 0)
      merged.back().bytes += r.bytes;
    else
      merged.push_back(r);
  }
  const size_t n = merged.size();
  int64_t total_bytes = 0;
  kern::InlineRanges inl;
  inl.n = 0;
  kern::RangeList list = {static_cast<int>(n), nullptr, nullptr, nullptr};
  DescriptorRing::Slot slot;
  const bool use_inline = inline_descriptors_ && n <= static_cast<size_t>(kern::INLINE_TENSORS);
  int64_t *h_vs, *h_off, *h_bytes;
  if (use_inline) {
    inl.n = static_cast<int>(n);
    h_vs = inl.vec_start;
    h_off = inl.byte_off;
    h_bytes = inl.bytes;
  } else {
    if ((n + 1) * 24 + 1024 > ring_.slot_bytes()) return false;
    slot = ring_.Acquire();
    int64_t *d_vs, *d_off, *d_bytes;
    h_vs = slot.Alloc<int64_t>(n + 1, &d_vs);
    h_off = slot.Alloc<int64_t>(n, &d_off);
    h_bytes = slot.Alloc<int64_t>(n, &d_bytes);
    list.vec_start = d_vs;
    list.byte_off = d_off;
    list.bytes = d_bytes;
  }
  int64_t v = 0;
  for (size_t i = 0; i < n; ++i) {
    h_vs[i] = v;
    h_off[i] = merged[i].off;
    h_bytes[i] = merged[i].bytes;
    v += (merged[i].bytes + 15) / 16;
    total_bytes += merged[i].bytes;
  }
  h_vs[n] = v;
  if (!use_inline) ring_.Commit(slot, stream_);
  const bool nvls = set.nvls && dtype != DataType::FLOAT64 && set.world >= 4 &&
                    forced_algo_ != "twoshot" && forced_algo_ != "oneshot";
  kern::SymmCtx ctx = MakeCtx(set, kern::EPOCHS_PER_LAUNCH);
  const int ctas = PickCtas(total_bytes);
  // Large messages: tiles of 64 KB drawn from a counter instead of one
  // slice per CTA (per-SM NVLink bandwidth is uneven on a two-die GPU).
  kern::TileSchedule sched = {nullptr, 0, 0};
  if (dynamic_min_bytes_ >= 0 && total_bytes >= dynamic_min_bytes_) {
    sched.counter = tile_counter_;
    sched.base = tile_base_;
    sched.tile_vecs = 4096;
    const int64_t per_rank = (v + set.world - 1) / set.world;
    const int64_t mine = std::max<int64_t>(
        0, std::min<int64_t>(per_rank, v - static_cast<int64_t>(set.rank) * per_rank));
    tile_base_ += static_cast<unsigned long long>((mine + sched.tile_vecs - 1) / sched.tile_vecs) +
                  static_cast<unsigned long long>(ctas);
  }
  host_trace::Mark("plan (in place)");
  cudaError_t err = kern::LaunchInplaceAllreduce(
      list, dtype, response.prescale * response.postscale,
      nvls || (forced_algo_ == "nvls" && set.nvls && dtype != DataType::FLOAT64),
      ctas, ctx, stream_, use_inline ? &inl : nullptr, &sched);
  host_trace::Mark("launch");
  if (!use_inline) ring_.Release(slot, stream_);
  *status = err == cudaSuccess
                ? Status::OK()
                : Status::UnknownError(std::string("in-place allreduce launch failed: ") +
                                       cudaGetErrorString(err));
  return true;
}

// A fused reducescatter response (several tensors of one dtype and one
// scaling) whose shards all fit one sender slot of the exchange region, none
// of them inside the symmetric heap: one launch for the whole group.
// *done stays false when the group does not qualify (the caller then runs the
// tensors one by one).
Status GpuOps::GroupedReducescatterPush(std::vector<TensorTableEntry>& entries, SymmSet& set,
                                        bool* done) {
  Timeline& tl = state_.timeline;
  const int n = set.world, me = set.rank;
  if (n <= 1 || set.xchg_bytes <= 0) return Status::OK();
  const TensorTableEntry& first = entries[0];
  const int64_t es = static_cast<int64_t>(DataTypeSize(first.dtype));
  const int64_t slot_bytes = set.xchg_bytes / n / STAGING_ALIGN * STAGING_ALIGN;
  struct Geo { int64_t base, extra, slice, longest_bytes; };
  std::vector<Geo> geo;
  int64_t need = 0;
  for (auto& e : entries) {
    if (e.dtype != first.dtype || e.prescale != first.prescale ||
        e.postscale != first.postscale || e.reduce_op != first.reduce_op)
      return Status::OK();
    int64_t heap_off = 0;
    if (e.input != nullptr && InSymmHeap(e.input, e.num_elements() * es, &heap_off))
      return Status::OK();
    int64_t rows = e.shape.dim_size(0), slice = 1;
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    Geo g;
    g.base = rows / n;
    g.extra = rows % n;
    g.slice = slice;
    g.longest_bytes = RoundUp((g.base + (g.extra ? 1 : 0)) * slice * es, STAGING_ALIGN);
    need += g.longest_bytes;
    geo.push_back(g);
  }
  if (need > slot_bytes || entries.size() > 2048) return Status::OK();

  for (size_t i = 0; i < entries.size(); ++i) {
    TensorTableEntry& e = entries[i];
    std::vector<int64_t> dims = e.shape.to_vector();
    dims[0] = geo[i].base + (me < geo[i].extra ? 1 : 0);
    tl.ActivityStart(e.name, HVD_ACT_ALLOCATE_OUTPUT);
    void* out = nullptr;
    Status st = e.context->AllocateOutput(TensorShape(dims), stream_, &out);
    tl.ActivityEnd(e.name);
    if (!st.ok()) return st;
    e.output = out;
  }

  const int ctas = PickCtas(need * n);
  const int64_t chunk = exchange_chunk_bytes_ / 256 * 256;
  DescriptorRing::Slot slot = ring_.Acquire();
  kern::RsGroupTensor* d_desc;
  kern::RsGroupTensor* h_desc = slot.Alloc<kern::RsGroupTensor>(entries.size(), &d_desc);
  if (h_desc == nullptr) {
    ring_.Release(slot, stream_);
    return Status::OK();  // too many tensors for a descriptor slot: one by one
  }
  int count = 0;
  int64_t off = 0, total_chunks = 0;
  for (size_t i = 0; i < entries.size(); ++i) {
    if (geo[i].longest_bytes == 0) continue;  // nothing to reduce
    kern::RsGroupTensor& d = h_desc[count++];
    d.in = entries[i].input;
    d.out = entries[i].output;
    d.base_rows = geo[i].base;
    d.extra_rows = geo[i].extra;
    d.row_elems = geo[i].slice;
    d.slot_off = off;
    const int64_t vecs = geo[i].longest_bytes / 16;
    d.slice_vecs = RoundUp((vecs + ctas - 1) / ctas, 16);
    total_chunks += (d.slice_vecs * 16 + chunk - 1) / chunk;
    off += geo[i].longest_bytes;
  }
  if (count == 0) {
    ring_.Release(slot, stream_);
    *done = true;
    return Status::OK();
  }
  ring_.Commit(slot, stream_);
  kern::RsGroupArgs a;
  std::memset(&a, 0, sizeof(a));
  a.tensors = d_desc;
  a.n_tensors = count;
  a.total_chunks = static_cast<uint32_t>(total_chunks);
  a.slot_bytes = slot_bytes;
  a.chunk_bytes = chunk;
  const uint32_t seq = ++set.xchg_seq;
  a.credit_wait = seq > 2 ? seq - 2 : 0;
  a.credit_post = seq;
  a.done_counter = xchg_done_counter_;
  xchg_done_base_ += static_cast<unsigned long long>(ctas);
  a.done_target = xchg_done_base_;
  kern::SymmCtx ctx = MakeCtx(set, static_cast<uint32_t>(total_chunks) + 1, set.xchg_off[seq & 1]);
  ActStart(entries, HVD_ACT_FUSED_KERNEL);
  cudaError_t err = kern::LaunchReducescatterPushGroup(a, first.dtype, first.prescale,
                                                       first.postscale, ctas, ctx, stream_);
  ActEnd(entries);
  ring_.Release(slot, stream_);
  if (err != cudaSuccess)
    return Status::UnknownError(std::string("grouped reducescatter launch failed: ") +
                                cudaGetErrorString(err));
  *done = true;
  return Status::OK();
}

Status GpuOps::SymmReducescatter(std::vector<TensorTableEntry>& entries,
                                 SymmSet& set) {
  Timeline& tl = state_.timeline;
  WaitForInputs(entries);
  if (entries.size() > 1) {
    bool done = false;
    Status st = GroupedReducescatterPush(entries, set, &done);
    if (!st.ok()) return st;
    if (done) return Complete(entries);
  }
  for (auto& e : entries) {
    const int64_t es = static_cast<int64_t>(DataTypeSize(e.dtype));
    const int n = set.world, me = set.rank;
    int64_t rows = e.shape.dim_size(0), slice = 1;
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    const int64_t base = rows / n, extra = rows % n;
    std::vector<int64_t> dims = e.shape.to_vector();
    dims[0] = base + (me < extra ? 1 : 0);
    tl.ActivityStart(e.name, HVD_ACT_ALLOCATE_OUTPUT);
    void* out = nullptr;
    Status st = e.context->AllocateOutput(TensorShape(dims), stream_, &out);
    tl.ActivityEnd(e.name);
    if (!st.ok()) return st;
    e.output = out;

    int64_t h_sb[SYMM_MAX_RANKS + 1];
    int64_t staged = 0;
    bool shards_aligned = true;
    for (int r = 0; r <= n; ++r) {
      h_sb[r] = (r * base + std::min<int64_t>(r, extra)) * slice;
      if ((h_sb[r] * es) & 15) shards_aligned = false;
      if (r > 0)
        staged += RoundUp((h_sb[r] - h_sb[r - 1]) * es, STAGING_ALIGN);
    }
    // An input inside the symmetric heap is reduced in place: no staging.
    int64_t sym_off = -1, heap_off = 0;
    if (n > 1 && shards_aligned && e.input != nullptr &&
        InSymmHeap(e.input, e.num_elements() * es, &heap_off) && (heap_off & 15) == 0)
      sym_off = heap_off;
    if (sym_off < 0 && n > 1 && set.xchg_bytes > 0) {
      // Ordinary memory: push every shard into its owner's exchange region,
      // one window of the shards per launch.
      const int64_t slot_bytes = set.xchg_bytes / n / STAGING_ALIGN * STAGING_ALIGN;
      const int64_t win = slot_bytes / es;
      const int64_t longest = (base + (extra ? 1 : 0)) * slice;
      const int64_t chunk = exchange_chunk_bytes_ / 256 * 256;
      ActStart(e.name, HVD_ACT_FUSED_KERNEL);
      for (int64_t lo = 0; lo < longest; lo += win) {
        const int64_t n_max = std::min(longest, lo + win) - lo;
        const int ctas = PickCtas(n_max * es * n);
        const int64_t vecs = (n_max * es + 15) / 16;
        kern::RsPushArgs a;
        std::memset(&a, 0, sizeof(a));
        for (int r = 0; r <= n; ++r) a.shard_begin[r] = h_sb[r];
        a.win_lo = lo;
        a.win_hi = lo + win;
        a.slot_bytes = slot_bytes;
        a.slice_vecs = RoundUp((vecs + ctas - 1) / ctas, 16);
        a.chunk_bytes = chunk;
        const uint32_t seq = ++set.xchg_seq;
        a.credit_wait = seq > 2 ? seq - 2 : 0;
        a.credit_post = seq;
        a.done_counter = xchg_done_counter_;
        xchg_done_base_ += static_cast<unsigned long long>(ctas);
        a.done_target = xchg_done_base_;
        const uint32_t epochs =
            static_cast<uint32_t>((a.slice_vecs * 16 + chunk - 1) / chunk) + 1;
        kern::SymmCtx ctx = MakeCtx(set, epochs, set.xchg_off[seq & 1]);
        cudaError_t err = kern::LaunchReducescatterPush(e.input, out, a, e.dtype, e.prescale,
                                                        e.postscale, ctas, ctx, stream_);
        if (err != cudaSuccess) {
          ActEnd(e.name);
          return Status::UnknownError(std::string("reducescatter launch failed: ") +
                                      cudaGetErrorString(err));
        }
      }
      ActEnd(e.name);
      continue;
    }
    if (sym_off < 0 && staged > static_cast<int64_t>(set.data_bytes))
      return Status::InvalidArgument(
          "reducescatter tensor '" + e.name + "' does not fit the symmetric "
          "staging buffer; raise HOROVOD_SYMM_BUFFER_MB.");
    // This kernel reads the shard bounds from device memory.
    DescriptorRing::Slot slot = ring_.Acquire();
    int64_t* d_sb;
    int64_t* ring_sb = slot.Alloc<int64_t>(n + 1, &d_sb);
    std::memcpy(ring_sb, h_sb, sizeof(int64_t) * (n + 1));
    ring_.Commit(slot, stream_);
    kern::SymmCtx ctx = MakeCtx(set, kern::EPOCHS_PER_LAUNCH);
    ActStart(e.name, HVD_ACT_FUSED_KERNEL);
    cudaError_t err = kern::LaunchFusedReducescatter(
        e.input, out, e.num_elements(), d_sb, e.dtype, sym_off >= 0 ? 1.0 : e.prescale,
        sym_off >= 0 ? e.prescale * e.postscale : e.postscale, set.nvls, PickCtas(staged),
        ctx, stream_, sym_off);
    ActEnd(e.name);
    ring_.Release(slot, stream_);
    if (err != cudaSuccess)
      return Status::UnknownError(std::string("reducescatter launch failed: ") +
                                  cudaGetErrorString(err));
  }
  return Complete(entries);
}

}  // namespace hvd
