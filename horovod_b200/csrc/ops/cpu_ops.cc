#include "cpu_ops.h"

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "../common/cpu_vector.h"
#include "../common/env.h"
#include "../common/fusion_buffer_manager.h"
#include "../common/global_state.h"
#include "../common/half.h"
#include "../common/logging.h"
#include "../common/process_set.h"

namespace hvd {

namespace {

double LoadAsDouble(const void* p, int64_t i, DataType t) {
  switch (t) {
  case DataType::FLOAT32: return static_cast<const float*>(p)[i];
  case DataType::FLOAT64: return static_cast<const double*>(p)[i];
  case DataType::FLOAT16: return HalfBitsToFloat(static_cast<const uint16_t*>(p)[i]);
  case DataType::BFLOAT16: return BF16BitsToFloat(static_cast<const uint16_t*>(p)[i]);
  default: return 0.0;
  }
}

void StoreFromDouble(void* p, int64_t i, DataType t, double v) {
  switch (t) {
  case DataType::FLOAT32: static_cast<float*>(p)[i] = static_cast<float>(v); break;
  case DataType::FLOAT64: static_cast<double*>(p)[i] = v; break;
  case DataType::FLOAT16:
    static_cast<uint16_t*>(p)[i] = FloatToHalfBits(static_cast<float>(v));
    break;
  case DataType::BFLOAT16:
    static_cast<uint16_t*>(p)[i] = FloatToBF16Bits(static_cast<float>(v));
    break;
  default: break;
  }
}

class CpuOps : public OpExecutor {
public:
  explicit CpuOps(GlobalState& s)
      : state_(s),
        buffers_([](size_t n) { return std::malloc(std::max<size_t>(n, 1)); },
                 [](void* p) { std::free(p); }) {}

  Status Execute(std::vector<TensorTableEntry>& entries,
                 const Response& response, ProcessSet& ps) override {
    switch (response.type) {
    case Response::ALLREDUCE: return Allreduce(entries, response, ps, false);
    case Response::ADASUM: return Allreduce(entries, response, ps, true);
    case Response::ALLGATHER: return Allgather(entries, response, ps);
    case Response::BROADCAST: return Broadcast(entries, ps);
    case Response::ALLTOALL: return Alltoall(entries, response, ps);
    case Response::REDUCESCATTER: return Reducescatter(entries, ps);
    default:
      return Status::InvalidArgument("hvd: unsupported CPU collective");
    }
  }

private:
  Status Allreduce(std::vector<TensorTableEntry>& entries,
                   const Response& response, ProcessSet& ps, bool adasum) {
    Timeline& tl = state_.timeline;
    const DataType dtype = response.dtype;
    const int64_t es = static_cast<int64_t>(DataTypeSize(dtype));
    const int64_t align_elems = std::max<int64_t>(1, FUSION_ALIGN_BYTES / es);
    // Layout of the fused buffer: each tensor starts on a 16-byte boundary.
    std::vector<int64_t> offsets(entries.size()), counts(entries.size());
    int64_t total = 0;
    for (size_t i = 0; i < entries.size(); ++i) {
      offsets[i] = total;
      counts[i] = entries[i].num_elements();
      total += RoundUp(counts[i], align_elems);
    }
    // A lone tensor is reduced without padding, on every rank alike (a rank
    // that joined has no output pointer but must send the same byte count).
    if (entries.size() == 1) total = counts[0];
    void* buf;
    bool in_place = entries.size() == 1 && entries[0].output != nullptr;
    if (in_place) {
      TensorTableEntry& e = entries[0];
      if (e.input != nullptr && e.input != e.output)
        std::memcpy(e.output, e.input, static_cast<size_t>(counts[0] * es));
      buf = e.output;
    } else {
      tl.ActivityStartAll(entries, HVD_ACT_MEMCPY_IN_FUSION_BUFFER);
      char* fusion = Fusion(static_cast<size_t>(total * es));
      std::memset(fusion, 0, static_cast<size_t>(total * es));
      for (size_t i = 0; i < entries.size(); ++i)
        if (entries[i].input != nullptr)
          std::memcpy(fusion + offsets[i] * es, entries[i].input,
                      static_cast<size_t>(counts[i] * es));
      buf = fusion;
      tl.ActivityEndAll(entries);
    }
    ScaleBufferCPU(buf, total, dtype, response.prescale);
    if (adasum) {
      tl.ActivityStartAll(entries, HVD_ACT_CPU_ADASUM);
      if (in_place) offsets[0] = 0;
      AdasumCPU(ps.comm, buf, dtype, offsets, counts, total);
    } else {
      tl.ActivityStartAll(entries, HVD_ACT_CPU_ALLREDUCE);
      if (ps.id == 0 && state_.hierarchy_usable &&
          state_.parameter_manager.HierarchicalAllreduce())
        HierarchicalAllreduce(buf, total, dtype, response.reduce_op);
      else
        ps.comm.Allreduce(buf, total, dtype, response.reduce_op);
    }
    tl.ActivityEndAll(entries);
    ScaleBufferCPU(buf, total, dtype, response.postscale);
    if (!in_place) {
      tl.ActivityStartAll(entries, HVD_ACT_MEMCPY_OUT_FUSION_BUFFER);
      for (size_t i = 0; i < entries.size(); ++i)
        if (entries[i].output != nullptr)
          std::memcpy(entries[i].output, static_cast<char*>(buf) + offsets[i] * es,
                      static_cast<size_t>(counts[i] * es));
      tl.ActivityEndAll(entries);
    }
    return Status::OK();
  }

  Status Allgather(std::vector<TensorTableEntry>& entries,
                   const Response& response, ProcessSet& ps) {
    Timeline& tl = state_.timeline;
    const int n = ps.comm.size();
    for (size_t i = 0; i < entries.size(); ++i) {
      TensorTableEntry& e = entries[i];
      int64_t slice = 1;
      for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
      int64_t slice_bytes = slice * static_cast<int64_t>(DataTypeSize(e.dtype));
      std::vector<int64_t> lens(n);
      int64_t rows = 0;
      for (int r = 0; r < n; ++r) {
        int64_t d0 = response.tensor_sizes[i * n + r];
        lens[r] = d0 * slice_bytes;
        rows += d0;
      }
      std::vector<int64_t> dims = e.shape.to_vector();
      dims[0] = rows;
      tl.ActivityStart(e.name, HVD_ACT_ALLOCATE_OUTPUT);
      void* out = nullptr;
      Status st = e.context->AllocateOutput(TensorShape(dims), nullptr, &out);
      tl.ActivityEnd(e.name);
      if (!st.ok()) return st;
      e.output = out;
      tl.ActivityStart(e.name, HVD_ACT_CPU_ALLGATHER);
      if (ps.id == 0 && state_.hierarchy_usable &&
          state_.parameter_manager.HierarchicalAllgather())
        HierarchicalAllgatherv(e.input, lens, out);
      else
        ps.comm.Allgatherv(e.input, lens, out);
      tl.ActivityEnd(e.name);
    }
    return Status::OK();
  }

  Status Broadcast(std::vector<TensorTableEntry>& entries, ProcessSet& ps) {
    Timeline& tl = state_.timeline;
    for (auto& e : entries) {
      size_t bytes = static_cast<size_t>(e.size_bytes());
      if (ps.comm.rank() == e.root_rank && e.input != e.output && bytes)
        std::memcpy(e.output, e.input, bytes);
      tl.ActivityStart(e.name, HVD_ACT_CPU_BCAST);
      ps.comm.Bcast(e.output, bytes, e.root_rank);
      tl.ActivityEnd(e.name);
    }
    return Status::OK();
  }

  Status Alltoall(std::vector<TensorTableEntry>& entries, const Response& response,
                  ProcessSet& ps) {
    Timeline& tl = state_.timeline;
    const int n = ps.comm.size();
    for (auto& e : entries) {
      int64_t slice = 1;
      for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
      int64_t slice_bytes = slice * static_cast<int64_t>(DataTypeSize(e.dtype));
      // Every rank tells every peer how many rows to expect.
      std::vector<int32_t> recv_splits(n);
      if (!AlltoallEvenRows(response, n, &recv_splits)) {
        std::vector<int64_t> four(n, 4);
        ps.comm.Alltoallv(e.splits.data(), four, recv_splits.data(), four);
      }
      std::vector<int64_t> send_lens(n), recv_lens(n);
      int64_t rows = 0;
      for (int r = 0; r < n; ++r) {
        send_lens[r] = e.splits[r] * slice_bytes;
        recv_lens[r] = recv_splits[r] * slice_bytes;
        rows += recv_splits[r];
      }
      std::vector<int64_t> dims = e.shape.to_vector();
      dims[0] = rows;
      tl.ActivityStart(e.name, HVD_ACT_ALLOCATE_OUTPUT);
      void* out = nullptr;
      Status st = e.context->AllocateOutput(TensorShape(dims), nullptr, &out);
      tl.ActivityEnd(e.name);
      if (!st.ok()) return st;
      e.output = out;
      e.context->SetReceivedSplits(recv_splits);
      tl.ActivityStart(e.name, HVD_ACT_CPU_ALLTOALL);
      ps.comm.Alltoallv(e.input, send_lens, out, recv_lens);
      tl.ActivityEnd(e.name);
    }
    return Status::OK();
  }

  Status Reducescatter(std::vector<TensorTableEntry>& entries, ProcessSet& ps) {
    Timeline& tl = state_.timeline;
    const int n = ps.comm.size(), me = ps.comm.rank();
    for (auto& e : entries) {
      int64_t es = static_cast<int64_t>(DataTypeSize(e.dtype));
      int64_t rows = e.shape.dim_size(0), slice = 1;
      for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
      // First (rows % n) ranks receive one extra row.
      int64_t base = rows / n, extra = rows % n;
      int64_t my_rows = base + (me < extra ? 1 : 0);
      int64_t my_start = me * base + std::min<int64_t>(me, extra);
      std::vector<int64_t> dims = e.shape.to_vector();
      dims[0] = my_rows;
      void* out = nullptr;
      Status st = e.context->AllocateOutput(TensorShape(dims), nullptr, &out);
      if (!st.ok()) return st;
      e.output = out;
      int64_t total = e.num_elements();
      char* fusion = Fusion(static_cast<size_t>(total * es));
      std::memcpy(fusion, e.input, static_cast<size_t>(total * es));
      ScaleBufferCPU(fusion, total, e.dtype, e.prescale);
      tl.ActivityStart(e.name, HVD_ACT_CPU_REDUCESCATTER);
      ps.comm.Allreduce(fusion, total, e.dtype, e.reduce_op);
      tl.ActivityEnd(e.name);
      std::memcpy(out, fusion + my_start * slice * es,
                  static_cast<size_t>(my_rows * slice * es));
      ScaleBufferCPU(out, my_rows * slice, e.dtype, e.postscale);
    }
    return Status::OK();
  }

  // Two-level allreduce: every host first reduce-scatters among its own
  // ranks (each ends up owning the host's partial sum of one shard), ranks
  // with the same local rank then allreduce their shard across hosts, and the
  // host finally allgathers the finished shards. Only 1 / local_size of the
  // data crosses hosts per rank.
  // Parity: horovod/common/ops/nccl_operations.cc:233-440 (same three steps).
  void HierarchicalAllreduce(void* buf, int64_t count, DataType dtype, ReduceOp op) {
    Comm& local = state_.local_comm;
    Comm& cross = state_.cross_comm;
    const int L = local.size(), me = local.rank();
    const int64_t es = static_cast<int64_t>(DataTypeSize(dtype));
    const int64_t base = count / L, extra = count % L;
    std::vector<int64_t> shard_bytes(L), mine_from_each(L);
    for (int r = 0; r < L; ++r) shard_bytes[r] = (base + (r < extra ? 1 : 0)) * es;
    const int64_t my_count = base + (me < extra ? 1 : 0);
    for (int r = 0; r < L; ++r) mine_from_each[r] = my_count * es;
    // Shard r of everybody's buffer goes to local rank r.
    std::vector<char> inbox(static_cast<size_t>(my_count * es) * L);
    local.Alltoallv(buf, shard_bytes, inbox.data(), mine_from_each);
    char* acc = inbox.data();
    for (int r = 1; r < L; ++r)
      ReduceInto(acc, inbox.data() + static_cast<size_t>(r) * my_count * es, my_count, dtype, op);
    cross.Allreduce(acc, my_count, dtype, op);
    local.Allgatherv(acc, shard_bytes, buf);
  }

  // Two-level allgather: blocks are first collected inside every host, then
  // whole host blocks travel between hosts (ranks are numbered host by host,
  // so the concatenation order is the global rank order).
  // Parity: horovod/common/ops/mpi_operations.cc hierarchical allgather.
  void HierarchicalAllgatherv(const void* in, const std::vector<int64_t>& lens, void* out) {
    Comm& local = state_.local_comm;
    Comm& cross = state_.cross_comm;
    const int L = local.size(), H = cross.size(), host = cross.rank();
    std::vector<int64_t> host_bytes(H, 0), host_start(H, 0);
    int64_t pos = 0;
    for (int h = 0; h < H; ++h) {
      host_start[h] = pos;
      for (int r = 0; r < L; ++r) host_bytes[h] += lens[static_cast<size_t>(h) * L + r];
      pos += host_bytes[h];
    }
    std::vector<int64_t> mine(lens.begin() + static_cast<size_t>(host) * L,
                              lens.begin() + static_cast<size_t>(host + 1) * L);
    std::vector<char> block(static_cast<size_t>(std::max<int64_t>(host_bytes[host], 1)));
    local.Allgatherv(in, mine, block.data());
    cross.Allgatherv(block.data(), host_bytes, out);
  }

  // The persistent host fusion buffer, sized for the fusion threshold in
  // effect (the autotuner may move it) or for the request if that is larger.
  char* Fusion(size_t bytes) {
    const size_t threshold =
        static_cast<size_t>(std::max<int64_t>(0, state_.parameter_manager.TensorFusionThresholdBytes()));
    return static_cast<char*>(buffers_.Get(CPU_DEVICE_ID, 0, bytes, threshold));
  }

  GlobalState& state_;
  FusionBufferManager buffers_;
};

}  // namespace

std::unique_ptr<OpExecutor> MakeCpuOps(GlobalState& state) {
  return std::unique_ptr<OpExecutor>(new CpuOps(state));
}

void AdasumCombineReference(const double* a, const double* b, double* out,
                            int64_t n) {
  double dot = 0, na = 0, nb = 0;
  for (int64_t i = 0; i < n; ++i) {
    dot += a[i] * b[i];
    na += a[i] * a[i];
    nb += b[i] * b[i];
  }
  const double tiny = std::sqrt(DBL_MIN);
  double ca = na >= tiny ? 1.0 - dot / (2 * na) : 1.0;
  double cb = nb >= tiny ? 1.0 - dot / (2 * nb) : 1.0;
  for (int64_t i = 0; i < n; ++i) out[i] = ca * a[i] + cb * b[i];
}

namespace {
// Exchanges with `peer` in pieces of at most HOROVOD_ADASUM_MPI_CHUNK_SIZE
// bytes (default 1 GiB; horovod/common/ops/adasum/adasum_mpi.cc:29-125 caps
// its MPI messages the same way). Both sides walk the same number of pieces:
// what one sends the other receives.
void ChunkedSendRecv(Comm& comm, int peer, const char* sbuf, size_t slen, char* rbuf,
                     size_t rlen) {
  static const size_t chunk =
      static_cast<size_t>(std::max<int64_t>(1, EnvInt(HVD_ENV_ADASUM_CHUNK, int64_t{1} << 30)));
  size_t so = 0, ro = 0;
  do {
    size_t sn = std::min(chunk, slen - so), rn = std::min(chunk, rlen - ro);
    comm.SendRecv(peer, sbuf + so, sn, peer, rbuf + ro, rn);
    so += sn;
    ro += rn;
  } while (so < slen || ro < rlen);
}
}  // namespace

void AdasumCPU(Comm& comm, void* buffer, DataType dtype,
               const std::vector<int64_t>& offsets,
               const std::vector<int64_t>& counts, int64_t total) {
  const int n = comm.size(), me = comm.rank();
  if (n <= 1 || total == 0) return;
  if ((n & (n - 1)) != 0)
    throw std::invalid_argument("Adasum needs a power-of-two number of ranks.");
  if (!IsFloatingPoint(dtype))
    throw std::invalid_argument("Adasum needs a floating point tensor.");
  const int64_t es = static_cast<int64_t>(DataTypeSize(dtype));
  char* data = static_cast<char*>(buffer);
  const size_t T = counts.size();
  const double tiny = std::sqrt(DBL_MIN);

  // Vector halving, distance doubling. [lo, hi) is the element range this
  // rank is still responsible for; it halves at every level.
  int64_t lo = 0, hi = total;
  std::vector<std::pair<int64_t, int64_t>> kept;  // ranges per level (for undo)
  std::vector<char> recv;
  for (int level = 1; level < n; level <<= 1) {
    int peer = me ^ level;
    bool lower = (me & level) == 0;
    int64_t mid = lo + (hi - lo) / 2;
    int64_t keep_lo = lower ? lo : mid, keep_hi = lower ? mid : hi;
    int64_t send_lo = lower ? mid : lo, send_hi = lower ? hi : mid;
    int64_t keep_n = keep_hi - keep_lo;
    recv.resize(static_cast<size_t>(keep_n * es));
    ChunkedSendRecv(comm, peer, data + send_lo * es,
                    static_cast<size_t>((send_hi - send_lo) * es), recv.data(),
                    static_cast<size_t>(keep_n * es));
    // "a" is always the lower group's vector, "b" the upper group's.
    const char* mine = data + keep_lo * es;
    const void* a = lower ? static_cast<const void*>(mine) : recv.data();
    const void* b = lower ? static_cast<const void*>(recv.data()) : mine;
    std::vector<double> stats(3 * T, 0.0);
    for (size_t t = 0; t < T; ++t) {
      int64_t s = std::max(offsets[t], keep_lo);
      int64_t e = std::min(offsets[t] + counts[t], keep_hi);
      double dot = 0, na = 0, nb = 0;
      if (e > s && dtype == DataType::FLOAT16) {
        HalfDotNorms(static_cast<const uint16_t*>(a) + (s - keep_lo),
                     static_cast<const uint16_t*>(b) + (s - keep_lo), e - s, &dot, &na, &nb);
      } else if (e > s && dtype == DataType::BFLOAT16) {
        BF16DotNorms(static_cast<const uint16_t*>(a) + (s - keep_lo),
                     static_cast<const uint16_t*>(b) + (s - keep_lo), e - s, &dot, &na, &nb);
      } else {
        for (int64_t i = s; i < e; ++i) {
          double x = LoadAsDouble(a, i - keep_lo, dtype);
          double y = LoadAsDouble(b, i - keep_lo, dtype);
          dot += x * y;
          na += x * x;
          nb += y * y;
        }
      }
      stats[3 * t] = dot;
      stats[3 * t + 1] = na;
      stats[3 * t + 2] = nb;
    }
    // Sum the partial products over the 2*level ranks that together hold the
    // two vectors being combined.
    int group = 2 * level;
    int first = me / group * group;
    std::vector<int> members(group);
    for (int i = 0; i < group; ++i) members[i] = first + i;
    Comm sub = comm.Subset(members);
    sub.Allreduce(stats.data(), static_cast<int64_t>(stats.size()),
                  DataType::FLOAT64, ReduceOp::SUM);
    for (size_t t = 0; t < T; ++t) {
      int64_t s = std::max(offsets[t], keep_lo);
      int64_t e = std::min(offsets[t] + counts[t], keep_hi);
      double dot = stats[3 * t], na = stats[3 * t + 1], nb = stats[3 * t + 2];
      double ca = na >= tiny ? 1.0 - dot / (2 * na) : 1.0;
      double cb = nb >= tiny ? 1.0 - dot / (2 * nb) : 1.0;
      if (e > s && (dtype == DataType::FLOAT16 || dtype == DataType::BFLOAT16)) {
        uint16_t* o = reinterpret_cast<uint16_t*>(data + keep_lo * es) + (s - keep_lo);
        const uint16_t* x16 = static_cast<const uint16_t*>(a) + (s - keep_lo);
        const uint16_t* y16 = static_cast<const uint16_t*>(b) + (s - keep_lo);
        if (dtype == DataType::FLOAT16)
          HalfScaledAdd(o, x16, y16, e - s, ca, cb);
        else
          BF16ScaledAdd(o, x16, y16, e - s, ca, cb);
        continue;
      }
      for (int64_t i = s; i < e; ++i) {
        double x = LoadAsDouble(a, i - keep_lo, dtype);
        double y = LoadAsDouble(b, i - keep_lo, dtype);
        StoreFromDouble(data + keep_lo * es, i - keep_lo, dtype, ca * x + cb * y);
      }
    }
    kept.emplace_back(lo, hi);
    lo = keep_lo;
    hi = keep_hi;
  }
  // Distance halving: hand the finished pieces back in reverse order.
  for (int level = n >> 1; level >= 1; level >>= 1) {
    int peer = me ^ level;
    auto range = kept.back();
    kept.pop_back();
    bool lower = (me & level) == 0;
    int64_t mid = range.first + (range.second - range.first) / 2;
    int64_t other_lo = lower ? mid : range.first;
    int64_t other_hi = lower ? range.second : mid;
    ChunkedSendRecv(comm, peer, data + lo * es, static_cast<size_t>((hi - lo) * es),
                    data + other_lo * es, static_cast<size_t>((other_hi - other_lo) * es));
    lo = range.first;
    hi = range.second;
  }
}

}  // namespace hvd
