// `_C.testing`: direct access to internal components for unit tests
// (software float conversions, wire format, Gaussian process, Bayesian
// optimisation, parameter manager, response cache, stall inspector, CPU
// reduction kernels, Adasum oracle).
#include <cstdlib>
#include <cstring>

#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../common/controller.h"
#include "../common/cpu_vector.h"
#include "../common/fusion_buffer_manager.h"
#include "../common/half.h"
#include "../common/message.h"
#include "../common/optim/bayesian_optimization.h"
#include "../common/parameter_manager.h"
#include "../common/response_cache.h"
#include "../common/stall_inspector.h"
#include "../common/tensor_queue.h"
#include "../kernels/kernels.h"
#include "../ops/cpu_ops.h"
#include "../ops/exchange_plan.h"
#include "../ops/nccl_api.h"
#include "../ops/nccl_comm_set.h"
#include "../transport/mesh.h"

namespace py = pybind11;

namespace hvd {

namespace {
// A stand-in for NCCL's error reporting: communicator `failing` starts to
// report an error at its `fail_at`-th query; aborts are counted.
struct FakeNcclState {
  int queries = 0, fail_at = 0, aborted = 0, destroyed = 0;
  ncclComm_t failing = nullptr;
};
FakeNcclState g_fake_nccl;
}  // namespace

void BindTesting(py::module_& root) {
  py::module_ m = root.def_submodule("testing", "internal components for unit tests");

  // Drives a FusionBufferManager over host memory with a list of (needed,
  // threshold) requests; returns the buffer size after each request and the
  // total number of (re)allocations.
  m.def("fusion_buffer_probe", [](const std::vector<std::pair<int64_t, int64_t>>& requests) {
    FusionBufferManager mgr([](size_t n) { return std::malloc(n ? n : 1); },
                            [](void* p) { std::free(p); });
    std::vector<int64_t> sizes;
    for (auto& r : requests) {
      void* p = mgr.Get(-1, 0, static_cast<size_t>(r.first), static_cast<size_t>(r.second));
      if (p != nullptr && r.first > 0) std::memset(p, 0xab, static_cast<size_t>(r.first));
      sizes.push_back(static_cast<int64_t>(mgr.SizeOf(-1, 0)));
    }
    return std::make_pair(sizes, mgr.reallocations());
  });
  m.def("cpu_has_f16c", &CpuHasF16C);
  m.def("cpu_vector_force_scalar", &CpuVectorForceScalar);
  // (a, b as uint16 bit patterns) -> (dot, |a|^2, |b|^2) and ca * a + cb * b.
  m.def("dot_norms_16", [](py::bytes a, py::bytes b, bool half) {
    std::string sa = a, sb = b;
    double dot = 0, na = 0, nb = 0;
    const int64_t n = static_cast<int64_t>(sa.size() / 2);
    auto* pa = reinterpret_cast<const uint16_t*>(sa.data());
    auto* pb = reinterpret_cast<const uint16_t*>(sb.data());
    if (half) HalfDotNorms(pa, pb, n, &dot, &na, &nb);
    else BF16DotNorms(pa, pb, n, &dot, &na, &nb);
    return std::make_tuple(dot, na, nb);
  });
  m.def("scaled_add_16", [](py::bytes a, py::bytes b, double ca, double cb, bool half) {
    std::string sa = a, sb = b;
    const int64_t n = static_cast<int64_t>(sa.size() / 2);
    std::string out(sa.size(), '\0');
    auto* pa = reinterpret_cast<const uint16_t*>(sa.data());
    auto* pb = reinterpret_cast<const uint16_t*>(sb.data());
    auto* po = reinterpret_cast<uint16_t*>(&out[0]);
    if (half) HalfScaledAdd(po, pa, pb, n, ca, cb);
    else BF16ScaledAdd(po, pa, pb, n, ca, cb);
    return py::bytes(out);
  });
  m.def("float_to_half_bits", &FloatToHalfBits);
  m.def("half_bits_to_float", &HalfBitsToFloat);
  m.def("float_to_bf16_bits", &FloatToBF16Bits);
  m.def("bf16_bits_to_float", &BF16BitsToFloat);

  // dst (op)= src on raw buffers given as Python bytes; returns new bytes.
  m.def("reduce_into", [](py::bytes dst, py::bytes src, int64_t count, int dtype, int op) {
    std::string d = dst, s = src;
    ReduceInto(&d[0], s.data(), count, static_cast<DataType>(dtype),
               static_cast<ReduceOp>(op));
    return py::bytes(d);
  });
  m.def("scale_buffer", [](py::bytes buf, int64_t count, int dtype, double factor) {
    std::string d = buf;
    ScaleBufferCPU(&d[0], count, static_cast<DataType>(dtype), factor);
    return py::bytes(d);
  });
  m.def("adasum_pair", [](const std::vector<double>& a, const std::vector<double>& b) {
    std::vector<double> out(a.size());
    AdasumCombineReference(a.data(), b.data(), out.data(), static_cast<int64_t>(a.size()));
    return out;
  });

  // Wire format round trip: builds a request/response list, serialises,
  // parses, and returns a few fields back.
  m.def("wire_roundtrip", [](const std::string& name, const std::vector<int64_t>& shape,
                             int dtype, double pre, double post) {
    Request q;
    q.request_rank = 3;
    q.type = Request::ALLGATHER;
    q.dtype = static_cast<DataType>(dtype);
    q.name = name;
    q.root_rank = 2;
    q.device = 1;
    q.group_id = 7;
    q.reduce_op = ReduceOp::MAX;
    q.shape = shape;
    q.prescale = pre;
    q.postscale = post;
    RequestList rl;
    rl.requests.push_back(q);
    rl.shutdown = true;
    std::string blob = rl.Serialize();
    RequestList back = RequestList::Parse(blob.data(), blob.size());
    const Request& r = back.requests.at(0);
    Response p;
    p.type = Response::ERROR;
    p.names = {name, name + "2"};
    p.error_message = "boom";
    p.devices = {0, 1};
    p.tensor_sizes = {5, 6, 7};
    p.last_joined_rank = 4;
    ResponseList pl;
    pl.responses.push_back(p);
    std::string pblob = pl.Serialize();
    ResponseList pback = ResponseList::Parse(pblob.data(), pblob.size());
    const Response& pr = pback.responses.at(0);
    return py::make_tuple(r.name, r.shape, static_cast<int>(r.dtype), r.prescale, r.postscale,
                          r.request_rank, static_cast<int>(r.type), r.root_rank, r.device,
                          r.group_id, static_cast<int>(r.reduce_op), back.shutdown,
                          pr.names, pr.error_message, pr.tensor_sizes, pr.last_joined_rank,
                          static_cast<int>(pr.type), blob.size());
  });
  // Fusion policy on a list of single-tensor responses given as tuples
  // (type, name, elements, dtype, prescale, postscale, root_rank); sizes follow
  // the reduction rule (each tensor rounded up to 16 bytes). Returns the
  // fused groups as lists of names, in execution order.
  m.def("fuse_responses", [](const std::vector<std::tuple<int, std::string, int64_t, int, double,
                                                          double, int>>& items,
                             int64_t threshold) {
    std::deque<Response> q;
    for (auto& it : items) {
      Response r;
      r.type = static_cast<Response::Type>(std::get<0>(it));
      r.names.push_back(std::get<1>(it));
      r.tensor_sizes.push_back(std::get<2>(it));
      r.dtype = static_cast<DataType>(std::get<3>(it));
      r.wire_dtype = r.dtype;
      r.prescale = std::get<4>(it);
      r.postscale = std::get<5>(it);
      r.root_rank = std::get<6>(it);
      r.reduce_op = ReduceOp::SUM;
      r.devices = {CPU_DEVICE_ID, CPU_DEVICE_ID};
      q.push_back(std::move(r));
    }
    ResponseList out;
    FuseResponseQueue(q, threshold, [](const Response& r) {
      int64_t es = static_cast<int64_t>(DataTypeSize(r.dtype)), total = 0;
      for (auto n : r.tensor_sizes) total += (n * es + 15) / 16 * 16;
      return total;
    }, out);
    std::vector<std::vector<std::string>> groups;
    for (auto& r : out.responses) groups.push_back(r.names);
    return groups;
  });
  // The wait of an elastic job for a device collective, on fakes: `comms`
  // communicators, of which number `failing` (or none: -1) reports an error
  // from its `fail_at`-th query on; the device work is done after
  // `ready_after` polls, or `ready_after_abort` polls after an abort.
  // Returns (ok, message, polls, queries, aborted, set empty, set failed,
  // destroyed by the final DestroyAll).
  m.def("nccl_async_wait", [](int comms, int failing, int fail_at, int ready_after,
                              int ready_after_abort) {
    g_fake_nccl = FakeNcclState();
    g_fake_nccl.fail_at = fail_at;
    NcclApi api{};
    api.CommGetAsyncError = [](ncclComm_t c, ncclResult_t* out) {
      if (c == g_fake_nccl.failing) ++g_fake_nccl.queries;
      *out = (c == g_fake_nccl.failing && g_fake_nccl.queries >= g_fake_nccl.fail_at)
                 ? ncclSystemError
                 : ncclSuccess;
      return ncclSuccess;
    };
    api.CommAbort = [](ncclComm_t) {
      ++g_fake_nccl.aborted;
      return ncclSuccess;
    };
    api.CommDestroy = [](ncclComm_t) {
      ++g_fake_nccl.destroyed;
      return ncclSuccess;
    };
    api.GetErrorString = [](ncclResult_t) -> const char* { return "peer is gone (fake)"; };
    NcclCommSet set(&api);
    for (int i = 0; i < comms; ++i)
      set.Put(i, reinterpret_cast<void*>(static_cast<uintptr_t>(0x1000 + i)));
    if (failing >= 0)
      g_fake_nccl.failing = reinterpret_cast<ncclComm_t>(static_cast<uintptr_t>(0x1000 + failing));
    int polls = 0, polls_after_abort = 0;
    Status st = WaitPolling(
        [&] {
          ++polls;
          if (g_fake_nccl.aborted > 0) return ++polls_after_abort >= ready_after_abort ? 1 : 0;
          return polls >= ready_after ? 1 : 0;
        },
        [&] { return set.CheckAsyncErrors(); }, std::chrono::microseconds(50),
        std::chrono::milliseconds(200));
    bool empty = set.empty(), failed = set.failed();
    int aborted = g_fake_nccl.aborted;
    set.DestroyAll();
    return py::make_tuple(st.ok(), st.reason(), polls, g_fake_nccl.queries, aborted, empty, failed,
                          g_fake_nccl.destroyed, set.failed());
  });
  m.def("affinity_core", [](const std::string& spec, int local_rank) {
    return AffinityCore(spec, local_rank);
  }, "Core that a HOROVOD_THREAD_AFFINITY value names for a local rank (-1: none).");
  // The exchange planner on plain numbers: blocks are (src_rank, dst_rank,
  // src address or 0, dst address or 0, bytes) as rank `rank` sees them;
  // returns one entry per round: (stage segments (src, self_dst, off, bytes,
  // dst), pull segments (dst, off, bytes, src_rank, sig_rank, chunks published
  // before), round_bytes, epochs). Addresses are opaque integers here, so a
  // test can replay the copies on arrays of its own.
  m.def("plan_exchange", [](const std::vector<std::tuple<int, int, uint64_t, uint64_t, int64_t>>&
                                blocks,
                            int rank, int world, int64_t region_bytes, bool push, int ctas,
                            int64_t chunk_bytes) {
    std::vector<ExchangeBlock> bl;
    for (auto& b : blocks) {
      ExchangeBlock e;
      e.src_rank = std::get<0>(b);
      e.dst_rank = std::get<1>(b);
      e.src = reinterpret_cast<const char*>(static_cast<uintptr_t>(std::get<2>(b)));
      e.dst = reinterpret_cast<char*>(static_cast<uintptr_t>(std::get<3>(b)));
      e.bytes = std::get<4>(b);
      bl.push_back(e);
    }
    py::list rounds;
    PlanExchangeRounds(bl, rank, world, region_bytes, push,
                       [&](const std::vector<ExchangeStageSeg>& stage,
                           const std::vector<ExchangePullSeg>& pull, int64_t round_bytes,
                           const std::vector<ExchangeRoundBlock>& round) {
      const ExchangeRoundSync rs = ComputeExchangeRoundSync(round, world, ctas, chunk_bytes);
      py::list st, pl;
      for (auto& g : stage)
        st.append(py::make_tuple(reinterpret_cast<uintptr_t>(g.src),
                                 reinterpret_cast<uintptr_t>(g.self_dst), g.off, g.bytes, g.dst));
      for (auto& g : pull)
        pl.append(py::make_tuple(reinterpret_cast<uintptr_t>(g.dst), g.off, g.bytes, g.src_rank,
                                 g.sig_rank, rs.before[g.block]));
      rounds.append(py::make_tuple(st, pl, round_bytes, rs.done_epochs));
    });
    return rounds;
  });
  m.def("wire_parse_garbage", [](py::bytes data) {
    std::string s = data;
    try {
      RequestList::Parse(s.data(), s.size());
    } catch (const std::exception&) {
      return false;
    }
    return true;
  });

  py::class_<GaussianProcess>(m, "GaussianProcess")
      .def(py::init<double>(), py::arg("alpha") = 1e-6)
      .def("fit", &GaussianProcess::Fit)
      .def("predict", [](const GaussianProcess& gp, const std::vector<double>& x) {
        double mean, sd;
        gp.Predict(x, &mean, &sd);
        return py::make_tuple(mean, sd);
      })
      .def_property_readonly("length_scale", &GaussianProcess::length_scale);

  py::class_<BayesianOptimization>(m, "BayesianOptimization")
      .def(py::init<std::vector<std::pair<double, double>>, double, double, uint64_t>(),
           py::arg("bounds"), py::arg("alpha") = 0.8, py::arg("xi") = 0.01,
           py::arg("seed") = 0)
      .def("add_sample", &BayesianOptimization::AddSample)
      .def("next_sample", &BayesianOptimization::NextSample)
      .def("best_x", &BayesianOptimization::best_x)
      .def("best_y", &BayesianOptimization::best_y);

  py::class_<ParameterManager>(m, "ParameterManager")
      .def(py::init<>())
      .def("initialize", &ParameterManager::Initialize)
      .def("set_auto_tuning", &ParameterManager::SetAutoTuning)
      .def("is_auto_tuning", &ParameterManager::IsAutoTuning)
      .def("set_warmup_samples", &ParameterManager::SetWarmupSamples)
      .def("set_steps_per_sample", &ParameterManager::SetStepsPerSample)
      .def("set_bayes_opt_max_samples", &ParameterManager::SetBayesOptMaxSamples)
      .def("set_cache_enabled", &ParameterManager::SetCacheEnabled, py::arg("v"),
           py::arg("fixed") = false)
      .def("set_hierarchical_allreduce", &ParameterManager::SetHierarchicalAllreduce,
           py::arg("v"), py::arg("fixed") = false)
      .def("set_hierarchical_allgather", &ParameterManager::SetHierarchicalAllgather,
           py::arg("v"), py::arg("fixed") = false)
      .def("set_fusion_threshold", &ParameterManager::SetTensorFusionThresholdBytes,
           py::arg("v"), py::arg("fixed") = false)
      .def("set_cycle_time_ms", &ParameterManager::SetCycleTimeMs, py::arg("v"),
           py::arg("fixed") = false)
      .def("update", &ParameterManager::Update)
      .def("fusion_threshold", &ParameterManager::TensorFusionThresholdBytes)
      .def("cycle_time_ms", &ParameterManager::CycleTimeMs)
      .def("cache_enabled", &ParameterManager::CacheEnabled)
      .def("samples_taken", &ParameterManager::samples_taken);

  // Response cache driven with synthetic allreduce requests.
  struct CacheHarness {
    ResponseCache cache;
    TensorQueue queue;
    Request MakeRequest(const std::string& name, const std::vector<int64_t>& shape, int dtype) {
      Request q;
      q.type = Request::ALLREDUCE;
      q.name = name;
      q.shape = shape;
      q.dtype = static_cast<DataType>(dtype);
      q.device = CPU_DEVICE_ID;
      return q;
    }
  };
  py::class_<CacheHarness>(m, "CacheHarness")
      .def(py::init<>())
      .def("set_capacity", [](CacheHarness& h, uint32_t c) { h.cache.set_capacity(c); })
      .def("cached", [](CacheHarness& h, const std::string& name,
                        const std::vector<int64_t>& shape, int dtype) {
        return static_cast<int>(h.cache.cached(h.MakeRequest(name, shape, dtype)));
      })
      .def("put", [](CacheHarness& h, const std::string& name,
                     const std::vector<int64_t>& shape, int dtype) {
        // The cache reads the shape from the pending entry.
        TensorTableEntry e;
        e.name = name;
        e.shape = TensorShape(shape);
        e.dtype = static_cast<DataType>(dtype);
        Request q = h.MakeRequest(name, shape, dtype);
        h.queue.AddToTensorQueue(e, q);
        Response r;
        r.type = Response::ALLREDUCE;
        r.names = {name};
        r.dtype = e.dtype;
        r.devices = {CPU_DEVICE_ID};
        r.tensor_sizes = {e.shape.num_elements()};
        h.cache.put(r, h.queue, false);
        std::vector<TensorTableEntry> drop;
        h.queue.GetTensorEntriesFromResponse(r, drop, false);
        h.cache.update_cache_bits();
      })
      .def("bit", [](CacheHarness& h, const std::string& name) {
        return h.cache.peek_cache_bit(name);
      })
      .def("touch", [](CacheHarness& h, uint32_t bit) {
        std::string n = h.cache.get_response(bit).names[0];
        h.cache.update_cache_bits();
        return n;
      })
      .def("erase", [](CacheHarness& h, uint32_t bit) {
        h.cache.erase_response(bit);
        h.cache.update_cache_bits();
      })
      .def("num_bits", [](CacheHarness& h) { return h.cache.num_active_bits(); })
      .def("has", [](CacheHarness& h, const std::string& n) { return h.cache.has_name(n); });

  // Cache coordinator: sync() over an in-process "allreduce" across the
  // given per-rank inputs. Each rank: (hits, invalid bits, shutdown, uncached).
  m.def("coordinate", [](size_t nbits,
                         const std::vector<std::tuple<std::vector<uint32_t>,
                                                      std::vector<uint32_t>, bool, bool>>& ranks) {
    // Two passes: collect every rank's words, reduce, hand the result back.
    std::vector<std::vector<std::vector<uint64_t>>> calls(ranks.size());
    std::vector<CacheCoordinator> ccs;
    for (auto& r : ranks) {
      CacheCoordinator cc(nbits);
      for (auto b : std::get<0>(r)) cc.record_hit(b);
      for (auto b : std::get<1>(r)) cc.record_invalid_bit(b);
      cc.set_should_shut_down(std::get<2>(r));
      cc.set_uncached_in_queue(std::get<3>(r));
      ccs.push_back(cc);
    }
    // First discover each rank's words by running sync with a recorder.
    std::vector<std::vector<uint64_t>> reduced;  // per call index
    for (int pass = 0; pass < 2; ++pass) {
      std::vector<CacheCoordinator> work = ccs;
      for (size_t i = 0; i < work.size(); ++i) {
        size_t call = 0;
        work[i].sync([&](uint64_t* w, size_t n, bool is_and) {
          if (pass == 0) {
            if (reduced.size() <= call) reduced.emplace_back(w, w + n);
            else
              for (size_t k = 0; k < n; ++k)
                reduced[call][k] = is_and ? (reduced[call][k] & w[k]) : (reduced[call][k] | w[k]);
          }
          if (pass == 1 && call < reduced.size())
            for (size_t k = 0; k < n; ++k) w[k] = reduced[call][k];
          ++call;
        });
        if (pass == 1) ccs[i] = work[i];
      }
    }
    py::list out;
    for (auto& cc : ccs)
      out.append(py::make_tuple(std::vector<uint32_t>(cc.cache_hits().begin(), cc.cache_hits().end()),
                                std::vector<uint32_t>(cc.invalid_bits().begin(), cc.invalid_bits().end()),
                                cc.should_shut_down(), cc.uncached_in_queue()));
    return out;
  });

  struct StallHarness {
    ResponseCache cache;
    StallInspector inspector;
    StallHarness() : inspector(cache) {}
  };
  py::class_<StallHarness>(m, "StallHarness")
      .def(py::init<>())
      .def("configure", [](StallHarness& h, int warn_s, int shutdown_s) {
        h.inspector.SetStallWarningTimeSeconds(warn_s);
        h.inspector.SetStallShutdownTimeSeconds(shutdown_s);
      })
      .def("record", [](StallHarness& h, const std::string& name, int rank, int size) {
        h.inspector.RecordUncachedTensorStart(name, rank, size);
      })
      .def("remove", [](StallHarness& h, const std::string& name) {
        h.inspector.RemoveUncachedTensor(name);
      })
      .def("check", [](StallHarness& h, const std::vector<int>& global_ranks) {
        bool shutdown = h.inspector.CheckForStalledTensors(global_ranks);
        return py::make_tuple(shutdown, h.inspector.last_report());
      });
}

}  // namespace hvd
