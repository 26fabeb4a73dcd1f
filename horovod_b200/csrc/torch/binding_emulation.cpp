// Several ranks on ONE GPU, for tests of the cross-rank kernel protocols on a
// box with a single GPU. Every "rank" gets its own slice of one device
// allocation (staging / exchange region, flag words, completion counter) and
// a SymmCtx whose peer pointers lead to the other ranks' slices; the kernels
// of all ranks then run as ONE cooperative launch (grid = CTAs per rank x
// ranks), so their CTAs are resident together and can wait for one another,
// which separate launches on one GPU could not guarantee. What runs is the
// production kernel body and, for the exchange ops, the production planner;
// only multimem (multicast over several GPUs) cannot be emulated.
// Every wait is bounded by `timeout_ms`; the functions return the kernel's
// status record with their results.
#include <torch/extension.h>

#include <pybind11/stl.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cstring>
#include <stdexcept>

#include "../common/common.h"
#include "../kernels/kernels.h"
#include "../ops/exchange_plan.h"
#include "../symm/symm_arena.h"

namespace py = pybind11;

namespace hvd {

namespace {

constexpr size_t kFlagWords =
    static_cast<size_t>(SYMM_FLAG_BANKS) * SYMM_MAX_RANKS * SYMM_MAX_BLOCKS;

DataType DTypeOf(const at::Tensor& t) {
  switch (t.scalar_type()) {
  case at::kFloat: return DataType::FLOAT32;
  case at::kBFloat16: return DataType::BFLOAT16;
  case at::kInt: return DataType::INT32;
  default: throw std::invalid_argument("emulation: dtype must be float32, bfloat16 or int32");
  }
}

void Check(cudaError_t e, const char* what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string("emulation: ") + what + ": " + cudaGetErrorString(e));
}

// The shared part of an emulated group: per-rank regions and flags in one
// zeroed device buffer, the host-mapped status record, the contexts.
struct Group {
  int world;
  at::Tensor memory;  // world x (region_bytes + flags + counter)
  int64_t region_bytes;
  kern::KernelStatus* status_host = nullptr;
  int* status_dev = nullptr;
  std::vector<kern::SymmCtx> ctx;
  std::vector<unsigned long long*> counters;

  Group(int world_, int64_t region_bytes_, int device, int timeout_ms)
      : world(world_), region_bytes(RoundUp(region_bytes_, 256)) {
    if (world < 1 || world > SYMM_MAX_RANKS)
      throw std::invalid_argument("emulation: 1 to 8 ranks");
    const int64_t flag_bytes = static_cast<int64_t>(kFlagWords * sizeof(uint32_t));
    const int64_t per_rank = region_bytes + flag_bytes + 256;
    memory = at::zeros({world * per_rank},
                       at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
    Check(cudaHostAlloc(reinterpret_cast<void**>(&status_host), sizeof(kern::KernelStatus),
                        cudaHostAllocMapped), "status record");
    std::memset(status_host, 0, sizeof(kern::KernelStatus));
    Check(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev), status_host, 0),
          "status pointer");
    char* base = static_cast<char*>(memory.data_ptr());
    ctx.resize(world);
    counters.resize(world);
    for (int r = 0; r < world; ++r) {
      kern::SymmCtx& c = ctx[r];
      std::memset(&c, 0, sizeof(c));
      c.rank = r;
      c.world = world;
      c.local = base + r * per_rank;
      c.flags_local = reinterpret_cast<uint32_t*>(base + r * per_rank + region_bytes);
      for (int p = 0; p < world; ++p) {
        c.peers[p] = base + p * per_rank;
        c.flags_peers[p] = reinterpret_cast<uint32_t*>(base + p * per_rank + region_bytes);
      }
      c.mc = nullptr;
      c.epoch = 0;
      c.timeout_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
      c.status = status_dev;
      counters[r] = reinterpret_cast<unsigned long long*>(base + r * per_rank + region_bytes +
                                                          flag_bytes);
    }
  }
  ~Group() {
    if (status_host != nullptr) cudaFreeHost(status_host);
  }
  py::tuple Status() const {
    return py::make_tuple(status_host->code, status_host->peer, status_host->phase,
                          status_host->block);
  }
};

// Copies a host array into a fresh device tensor and returns it (kept alive
// by the caller until the launch has finished).
template <typename T>
at::Tensor ToDevice(const std::vector<T>& host, int device) {
  at::Tensor t = at::empty({static_cast<int64_t>(std::max<size_t>(host.size(), 1) * sizeof(T))},
                           at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
  if (!host.empty())
    Check(cudaMemcpy(t.data_ptr(), host.data(), host.size() * sizeof(T),
                     cudaMemcpyHostToDevice), "descriptor copy");
  return t;
}

void CheckSameDevice(const std::vector<std::vector<at::Tensor>>& ranks, int* device) {
  if (ranks.empty() || ranks[0].empty()) throw std::invalid_argument("emulation: no tensors");
  *device = ranks[0][0].get_device();
  for (auto& list : ranks)
    for (auto& t : list)
      if (!t.is_cuda() || t.get_device() != *device || !t.is_contiguous())
        throw std::invalid_argument("emulation: contiguous tensors on one CUDA device");
}

}  // namespace

void BindEmulation(py::module_& m) {
  // In-place fused allreduce (sum) of every rank's tensor list, as the
  // one-shot or two-shot kernel would run it on `len(ranks)` GPUs.
  // sub_chunk_kb > 0 pipelines the two-shot variant over sub-chunks.
  // Returns the status record (code, peer, phase, block).
  m.def("emulated_allreduce", [](std::vector<std::vector<at::Tensor>> ranks,
                                 const std::string& algo, int ctas, int sub_chunk_kb,
                                 double prescale, double postscale, bool bf16_wire,
                                 int launches, int timeout_ms) {
    int device = 0;
    CheckSameDevice(ranks, &device);
    c10::cuda::CUDAGuard guard(device);
    const int world = static_cast<int>(ranks.size());
    const DataType dtype = DTypeOf(ranks[0][0]);
    const DataType wire = bf16_wire ? DataType::BFLOAT16 : dtype;
    if (bf16_wire && dtype != DataType::FLOAT32)
      throw std::invalid_argument("emulation: a bf16 wire needs float32 tensors");
    const int64_t ws = static_cast<int64_t>(DataTypeSize(wire));
    const int64_t align_elems = FUSION_ALIGN_BYTES / ws;
    const size_t n = ranks[0].size();
    std::vector<int64_t> offsets(n + 1, 0), counts(n);
    for (size_t i = 0; i < n; ++i) {
      counts[i] = ranks[0][i].numel();
      offsets[i + 1] = offsets[i] + RoundUp(counts[i], align_elems);
      for (auto& list : ranks)
        if (list.size() != n || list[i].numel() != counts[i] || DTypeOf(list[i]) != dtype)
          throw std::invalid_argument("emulation: every rank passes the same shapes and dtype");
    }
    const int64_t bytes = offsets[n] * ws;
    Group group(world, bytes + 4096, device, timeout_ms);
    const kern::Algo a = algo == "oneshot" ? kern::Algo::ONESHOT : kern::Algo::TWOSHOT;
    if (algo != "oneshot" && algo != "twoshot")
      throw std::invalid_argument("emulation: algo is oneshot or twoshot");
    const int64_t sub_vecs = a == kern::Algo::TWOSHOT ? int64_t(sub_chunk_kb) * 1024 / 16 : 0;
    const uint32_t epochs =
        a == kern::Algo::TWOSHOT
            ? std::max(kern::EPOCHS_PER_LAUNCH,
                       kern::FusedAllreduceEpochs(bytes / 16, world, ctas, sub_vecs))
            : kern::EPOCHS_PER_LAUNCH;
    at::Tensor d_off = ToDevice(offsets, device), d_cnt = ToDevice(counts, device);
    std::vector<at::Tensor> keep;
    std::vector<kern::EmuAllreduceRank> host(world);
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(device).stream();
    for (int launch = 0; launch < launches; ++launch) {
      for (int r = 0; r < world; ++r) {
        std::vector<const void*> in(n);
        for (size_t i = 0; i < n; ++i) in[i] = ranks[r][i].data_ptr();
        at::Tensor d_in = ToDevice(in, device);
        keep.push_back(d_in);
        host[r].tl.n = static_cast<int>(n);
        host[r].tl.offsets = static_cast<const int64_t*>(d_off.data_ptr());
        host[r].tl.counts = static_cast<const int64_t*>(d_cnt.data_ptr());
        host[r].tl.in = static_cast<const void* const*>(d_in.data_ptr());
        host[r].tl.out = static_cast<void* const*>(d_in.data_ptr());
        host[r].ctx = group.ctx[r];
        host[r].ctx.epoch = static_cast<uint32_t>(launch) * epochs;
        host[r].ctx.sub_chunk_vecs = sub_vecs;
      }
      at::Tensor d_ranks = ToDevice(host, device);
      keep.push_back(d_ranks);
      Check(kern::LaunchFusedAllreduceEmulated(
                static_cast<const kern::EmuAllreduceRank*>(d_ranks.data_ptr()), world, dtype,
                wire, prescale, postscale, a, ctas, stream),
            "allreduce launch");
    }
    Check(cudaStreamSynchronize(stream), "allreduce kernel");
    return group.Status();
  }, py::arg("ranks"), py::arg("algo") = "twoshot", py::arg("ctas") = 4,
     py::arg("sub_chunk_kb") = 0, py::arg("prescale") = 1.0, py::arg("postscale") = 1.0,
     py::arg("bf16_wire") = false, py::arg("launches") = 1, py::arg("timeout_ms") = 2000);

  // Reduce-scatter of one tensor per rank (same shape everywhere) by the push
  // kernel: returns (list of each rank's shard, status record).
  m.def("emulated_reducescatter", [](std::vector<at::Tensor> inputs, int ctas, int chunk_kb,
                                     double prescale, double postscale, int64_t region_kb,
                                     int timeout_ms) {
    std::vector<std::vector<at::Tensor>> as_lists;
    for (auto& t : inputs) as_lists.push_back({t});
    int device = 0;
    CheckSameDevice(as_lists, &device);
    c10::cuda::CUDAGuard guard(device);
    const int world = static_cast<int>(inputs.size());
    const DataType dtype = DTypeOf(inputs[0]);
    const int64_t es = static_cast<int64_t>(DataTypeSize(dtype));
    const at::Tensor& first = inputs[0];
    if (first.dim() < 1) throw std::invalid_argument("emulation: tensors need a first dimension");
    for (auto& t : inputs)
      if (t.sizes() != first.sizes() || DTypeOf(t) != dtype)
        throw std::invalid_argument("emulation: every rank passes the same shape and dtype");
    const int64_t rows = first.size(0), slice = rows > 0 ? first.numel() / rows : 0;
    const int64_t base = rows / world, extra = rows % world;
    std::vector<int64_t> sb(world + 1);
    for (int r = 0; r <= world; ++r) sb[r] = (r * base + std::min<int64_t>(r, extra)) * slice;
    const int64_t region_bytes = region_kb * 1024;
    const int64_t slot_bytes = region_bytes / world / 256 * 256;
    if (slot_bytes < 4096) throw std::invalid_argument("emulation: region too small");
    Group group(world, region_bytes, device, timeout_ms);
    std::vector<at::Tensor> outs;
    for (int r = 0; r < world; ++r) {
      std::vector<int64_t> dims = first.sizes().vec();
      dims[0] = base + (r < extra ? 1 : 0);
      outs.push_back(at::zeros(dims, first.options()));
    }
    const int64_t win = slot_bytes / es;
    const int64_t longest = (base + (extra ? 1 : 0)) * slice;
    const int64_t chunk = int64_t(chunk_kb) * 1024 / 256 * 256;
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(device).stream();
    std::vector<at::Tensor> keep;
    uint32_t epoch = 0, seq = 0;
    unsigned long long done_base = 0;
    // Windows of the shards, as the executor cuts them; every launch uses the
    // same region here, so its credit wait is the credit of the launch before.
    for (int64_t lo = 0; lo < longest; lo += win) {
      const int64_t n_max = std::min(longest, lo + win) - lo;
      const int64_t vecs = (n_max * es + 15) / 16;
      std::vector<kern::EmuRsPushRank> host(world);
      ++seq;
      done_base += static_cast<unsigned long long>(ctas);
      uint32_t epochs = 0;
      for (int r = 0; r < world; ++r) {
        kern::EmuRsPushRank& e = host[r];
        std::memset(&e, 0, sizeof(e));
        e.in = inputs[r].data_ptr();
        e.out = outs[r].data_ptr();
        for (int p = 0; p <= world; ++p) e.args.shard_begin[p] = sb[p];
        e.args.win_lo = lo;
        e.args.win_hi = lo + win;
        e.args.slot_bytes = slot_bytes;
        e.args.slice_vecs = RoundUp((vecs + ctas - 1) / ctas, 16);
        e.args.chunk_bytes = chunk;
        e.args.credit_wait = seq > 1 ? seq - 1 : 0;
        e.args.credit_post = seq;
        e.args.done_counter = group.counters[r];
        e.args.done_target = done_base;
        epochs = static_cast<uint32_t>((e.args.slice_vecs * 16 + chunk - 1) / chunk) + 1;
        e.ctx = group.ctx[r];
        e.ctx.epoch = epoch;
      }
      epoch += epochs;
      at::Tensor d_ranks = ToDevice(host, device);
      keep.push_back(d_ranks);
      Check(kern::LaunchReducescatterPushEmulated(
                static_cast<const kern::EmuRsPushRank*>(d_ranks.data_ptr()), world, dtype,
                prescale, postscale, ctas, stream),
            "reducescatter launch");
    }
    Check(cudaStreamSynchronize(stream), "reducescatter kernel");
    return py::make_tuple(outs, group.Status());
  }, py::arg("inputs"), py::arg("ctas") = 4, py::arg("chunk_kb") = 64,
     py::arg("prescale") = 1.0, py::arg("postscale") = 1.0, py::arg("region_kb") = 4096,
     py::arg("timeout_ms") = 2000);

  // Allgather (inputs[r] = rank r's rows), broadcast (root >= 0: inputs[root]
  // goes to everybody) or alltoall (splits[r][p] = rows rank r sends to rank
  // p) through the production planner and the exchange kernel. push: blocks
  // are stored into the receivers' regions instead of pulled from the
  // sender's. Returns (outputs per rank, status record).
  m.def("emulated_exchange", [](const std::string& op, std::vector<at::Tensor> inputs,
                                std::vector<std::vector<int64_t>> splits, int root, bool push,
                                int ctas, int chunk_kb, int64_t region_kb, int timeout_ms) {
    std::vector<std::vector<at::Tensor>> as_lists;
    for (auto& t : inputs) as_lists.push_back({t});
    int device = 0;
    CheckSameDevice(as_lists, &device);
    c10::cuda::CUDAGuard guard(device);
    const int world = static_cast<int>(inputs.size());
    const int64_t es = static_cast<int64_t>(inputs[0].element_size());
    auto slice_of = [&](const at::Tensor& t) {
      int64_t s = es;
      for (int d = 1; d < t.dim(); ++d) s *= t.size(d);
      return s;
    };
    const int64_t slice = slice_of(inputs[0]);
    // Outputs and, per rank, that rank's view of the global block list.
    std::vector<at::Tensor> outs(world);
    std::vector<std::vector<ExchangeBlock>> blocks(world);
    auto dims_with_rows = [&](int64_t rows) {
      std::vector<int64_t> d = inputs[0].sizes().vec();
      d[0] = rows;
      return d;
    };
    if (op == "allgather") {
      int64_t rows = 0;
      for (auto& t : inputs) rows += t.size(0);
      for (int me = 0; me < world; ++me) {
        outs[me] = at::zeros(dims_with_rows(rows), inputs[0].options());
        int64_t disp = 0;
        for (int r = 0; r < world; ++r) {
          ExchangeBlock b;
          b.src_rank = r;
          b.dst_rank = -1;
          b.src = r == me ? static_cast<const char*>(inputs[r].data_ptr()) : nullptr;
          b.dst = static_cast<char*>(outs[me].data_ptr()) + disp;
          b.bytes = inputs[r].size(0) * slice;
          disp += b.bytes;
          blocks[me].push_back(b);
        }
      }
    } else if (op == "broadcast") {
      if (root < 0 || root >= world) throw std::invalid_argument("emulation: bad root");
      for (int me = 0; me < world; ++me) {
        outs[me] = me == root ? inputs[root] : at::zeros_like(inputs[root]);
        ExchangeBlock b;
        b.src_rank = root;
        b.dst_rank = -1;
        b.src = static_cast<const char*>(inputs[root].data_ptr());
        b.dst = me == root ? nullptr : static_cast<char*>(outs[me].data_ptr());
        b.bytes = inputs[root].numel() * es;
        blocks[me].push_back(b);
      }
    } else if (op == "alltoall") {
      if (static_cast<int>(splits.size()) != world)
        throw std::invalid_argument("emulation: one split row per rank");
      for (int me = 0; me < world; ++me) {
        int64_t rows = 0;
        for (int r = 0; r < world; ++r) rows += splits[r][me];
        outs[me] = at::zeros(dims_with_rows(rows), inputs[0].options());
        std::vector<int64_t> send_off(world, 0), recv_off(world, 0);
        for (int p = 1; p < world; ++p) {
          send_off[p] = send_off[p - 1] + splits[me][p - 1] * slice;
          recv_off[p] = recv_off[p - 1] + splits[p - 1][me] * slice;
        }
        for (int r = 0; r < world; ++r) {
          for (int j = 1; j <= world; ++j) {
            const int p = (r + j) % world;
            ExchangeBlock b;
            b.src_rank = r;
            b.dst_rank = p;
            b.bytes = splits[r][p] * slice;
            b.src = r == me ? static_cast<const char*>(inputs[me].data_ptr()) + send_off[p]
                            : nullptr;
            b.dst = p == me ? static_cast<char*>(outs[me].data_ptr()) + recv_off[r] : nullptr;
            blocks[me].push_back(b);
          }
        }
      }
    } else {
      throw std::invalid_argument("emulation: op is allgather, broadcast or alltoall");
    }

    const int64_t region_bytes = region_kb * 1024;
    Group group(world, region_bytes, device, timeout_ms);
    // (A segment of up to 64 KB is one chunk of one CTA: chunks are at least that.)
    const int64_t chunk = std::max<int64_t>(64 * 1024, int64_t(chunk_kb) * 1024 / 256 * 256);
    // Rounds per rank from the production planner (the same count on every
    // rank, since the plan depends on shared data only).
    struct Round {
      std::vector<ExchangeStageSeg> stage;
      std::vector<ExchangePullSeg> pull;
      std::vector<ExchangeRoundBlock> blocks;
    };
    std::vector<std::vector<Round>> rounds(world);
    for (int me = 0; me < world; ++me)
      PlanExchangeRounds(blocks[me], me, world, region_bytes, push,
                         [&](const std::vector<ExchangeStageSeg>& s,
                             const std::vector<ExchangePullSeg>& p, int64_t,
                             const std::vector<ExchangeRoundBlock>& rb) {
                           rounds[me].push_back({s, p, rb});
                         });
    for (int me = 1; me < world; ++me)
      if (rounds[me].size() != rounds[0].size())
        throw std::runtime_error("emulation: ranks disagree on the number of rounds");

    cudaStream_t stream = c10::cuda::getCurrentCUDAStream(device).stream();
    std::vector<at::Tensor> keep;
    uint32_t epoch = 0, seq = 0;
    unsigned long long done_base = 0;
    for (size_t k = 0; k < rounds[0].size(); ++k) {
      const ExchangeRoundSync rs = ComputeExchangeRoundSync(rounds[0][k].blocks, world, ctas, chunk);
      ++seq;
      done_base += static_cast<unsigned long long>(ctas);
      std::vector<kern::EmuExchangeRank> host(world);
      for (int me = 0; me < world; ++me) {
        const Round& rd = rounds[me][k];
        const size_t ns = rd.stage.size(), np = rd.pull.size();
        std::vector<const void*> st_src(ns + 1);
        std::vector<void*> st_self(ns + 1), pl_dst(np + 1);
        std::vector<int64_t> st_off(ns + 1), st_bytes(ns + 1), pl_off(np + 1), pl_bytes(np + 1);
        std::vector<int32_t> st_dst(ns + 1), pl_src(np + 1), pl_sig(np + 1), pl_wait(np + 1);
        for (size_t i = 0; i < ns; ++i) {
          st_src[i] = rd.stage[i].src;
          st_self[i] = rd.stage[i].self_dst;
          st_off[i] = rd.stage[i].off;
          st_bytes[i] = rd.stage[i].bytes;
          st_dst[i] = rd.stage[i].dst;
        }
        for (size_t i = 0; i < np; ++i) {
          pl_dst[i] = rd.pull[i].dst;
          pl_off[i] = rd.pull[i].off;
          pl_bytes[i] = rd.pull[i].bytes;
          pl_src[i] = rd.pull[i].src_rank;
          pl_sig[i] = rd.pull[i].sig_rank;
          pl_wait[i] = static_cast<int32_t>(rs.before[rd.pull[i].block]);
        }
        at::Tensor a0 = ToDevice(st_src, device), a1 = ToDevice(st_self, device),
                   a2 = ToDevice(st_off, device), a3 = ToDevice(st_bytes, device),
                   a4 = ToDevice(st_dst, device), a5 = ToDevice(pl_dst, device),
                   a6 = ToDevice(pl_off, device), a7 = ToDevice(pl_bytes, device),
                   a8 = ToDevice(pl_src, device), a9 = ToDevice(pl_sig, device),
                   a10 = ToDevice(pl_wait, device);
        for (auto& t : {a0, a1, a2, a3, a4, a5, a6, a7, a8, a9, a10}) keep.push_back(t);
        kern::EmuExchangeRank& e = host[me];
        std::memset(&e, 0, sizeof(e));
        e.plan.n_stage = static_cast<int>(ns);
        e.plan.st_src = static_cast<const void**>(a0.data_ptr());
        e.plan.st_self = static_cast<void**>(a1.data_ptr());
        e.plan.st_off = static_cast<int64_t*>(a2.data_ptr());
        e.plan.st_bytes = static_cast<int64_t*>(a3.data_ptr());
        e.plan.st_dst = static_cast<int32_t*>(a4.data_ptr());
        e.plan.n_pull = static_cast<int>(np);
        e.plan.pl_dst = static_cast<void**>(a5.data_ptr());
        e.plan.pl_off = static_cast<int64_t*>(a6.data_ptr());
        e.plan.pl_bytes = static_cast<int64_t*>(a7.data_ptr());
        e.plan.pl_src = static_cast<int32_t*>(a8.data_ptr());
        e.plan.pl_sig = static_cast<int32_t*>(a9.data_ptr());
        e.plan.pl_wait = static_cast<int32_t*>(a10.data_ptr());
        e.sync.chunk_bytes = chunk;
        e.sync.done_epochs = rs.done_epochs;
        // One region here: a launch may overwrite it once every peer has
        // finished the launch before.
        e.sync.credit_wait = seq > 1 ? seq - 1 : 0;
        e.sync.credit_post = seq;
        e.sync.done_counter = group.counters[me];
        e.sync.done_target = done_base;
        e.ctx = group.ctx[me];
        e.ctx.epoch = epoch;
      }
      epoch += rs.done_epochs;
      at::Tensor d_ranks = ToDevice(host, device);
      keep.push_back(d_ranks);
      Check(kern::LaunchExchangeEmulated(
                static_cast<const kern::EmuExchangeRank*>(d_ranks.data_ptr()), world, ctas,
                stream),
            "exchange launch");
    }
    Check(cudaStreamSynchronize(stream), "exchange kernel");
    return py::make_tuple(outs, group.Status(), static_cast<int>(rounds[0].size()));
  }, py::arg("op"), py::arg("inputs"), py::arg("splits") = std::vector<std::vector<int64_t>>(),
     py::arg("root") = -1, py::arg("push") = false, py::arg("ctas") = 4,
     py::arg("chunk_kb") = 64, py::arg("region_kb") = 4096, py::arg("timeout_ms") = 2000);
}

}  // namespace hvd
