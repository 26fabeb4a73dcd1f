// PyTorch binding: turns torch tensors into table entries, records ready
// events on torch's current stream, hands out integer handles, and lets
// Python poll / wait on them. Waiting on a GPU op does not block the host on
// the GPU: once the background thread has launched the op, the caller's
// current stream is made to wait on the op's completion event.
//
// Parity: horovod/torch/mpi_ops_v2.cc:89-785 (Do* functions, poll,
// wait_and_clear, join), adapter_v2.cc:22-162 (tensor/context adapters,
// status -> exception mapping), ready_event.cc:51-99, handle_manager.cc
// :21-57. One pybind function per op serves every dtype and device.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime_api.h>

#include <atomic>
#include <condition_variable>
#include <mutex>
#include <unordered_map>

#include "../common/logging.h"
#include "../common/operations.h"
#include "../ops/gpu_ops.h"

namespace py = pybind11;

namespace hvd {
// Defined in binding_gpu.cpp: topology / symmetric-memory diagnostics and
// raw kernel entry points used by the GPU tests and benchmarks.
void BindGpuDiagnostics(py::module_& m);
// Defined in binding_testing.cpp.
void BindTesting(py::module_& m);
void BindModelOps(py::module_& m);
void BindEmulation(py::module_& m);

namespace {

DataType ToDataType(at::ScalarType t) {
  switch (t) {
  case at::kByte: return DataType::UINT8;
  case at::kChar: return DataType::INT8;
  case at::kShort: return DataType::INT16;
  case at::kInt: return DataType::INT32;
  case at::kLong: return DataType::INT64;
  case at::kHalf: return DataType::FLOAT16;
  case at::kFloat: return DataType::FLOAT32;
  case at::kDouble: return DataType::FLOAT64;
  case at::kBool: return DataType::BOOL;
  case at::kBFloat16: return DataType::BFLOAT16;
  case at::kUInt16: return DataType::UINT16;
  default:
    throw std::invalid_argument(std::string("Unsupported tensor dtype for a "
                                            "Horovod collective: ") +
                                c10::toString(t));
  }
}

int DeviceOf(const at::Tensor& t) {
  return t.is_cuda() ? static_cast<int>(t.get_device()) : CPU_DEVICE_ID;
}

// ---- ready events ---------------------------------------------------------

class EventPool {
public:
  cudaEvent_t Get(int device) {
    {
      std::lock_guard<std::mutex> l(mu_);
      auto& v = free_[device];
      if (!v.empty()) {
        cudaEvent_t e = v.back();
        v.pop_back();
        return e;
      }
    }
    c10::cuda::CUDAGuard guard(device);
    cudaEvent_t e;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess)
      throw std::runtime_error("hvd: cudaEventCreate failed");
    return e;
  }
  void Put(int device, cudaEvent_t e) {
    std::lock_guard<std::mutex> l(mu_);
    free_[device].push_back(e);
  }

private:
  std::mutex mu_;
  std::unordered_map<int, std::vector<cudaEvent_t>> free_;
};

EventPool& Events() {
  static EventPool* pool = new EventPool();  // outlives static destruction
  return *pool;
}

class TorchReadyEvent : public ReadyEvent {
public:
  explicit TorchReadyEvent(int device) : device_(device) {
    event_ = Events().Get(device);
    // The default stream's handle means "the default stream of the current
    // device", so that device must be current while the event is recorded.
    c10::cuda::CUDAGuard guard(device);
    auto stream = at::cuda::getCurrentCUDAStream(device);
    if (cudaEventRecord(event_, stream.stream()) != cudaSuccess)
      throw std::runtime_error("hvd: cudaEventRecord failed");
  }
  ~TorchReadyEvent() override { Events().Put(device_, event_); }
  bool Ready() const override { return cudaEventQuery(event_) == cudaSuccess; }
  void StreamWait(void* stream) const override {
    cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), event_, 0);
  }

private:
  int device_;
  cudaEvent_t event_;
};

// ---- handles --------------------------------------------------------------

struct HandleRecord {
  std::mutex mu;
  std::condition_variable cv;
  int pending = 1;  // callbacks still to arrive
  Status status;
  std::shared_ptr<void> done_event;
  int device = CPU_DEVICE_ID;
  std::vector<at::Tensor> inputs;   // kept alive until the op is done
  std::vector<at::Tensor> outputs;
  std::vector<int32_t> received_splits;
  bool has_splits = false;
  int32_t join_result = -1;
};

class HandleManager {
public:
  int Allocate(std::shared_ptr<HandleRecord> rec) {
    std::lock_guard<std::mutex> l(mu_);
    int h = next_++;
    table_[h] = std::move(rec);
    return h;
  }
  std::shared_ptr<HandleRecord> Get(int h) {
    std::lock_guard<std::mutex> l(mu_);
    auto it = table_.find(h);
    if (it == table_.end())
      throw std::invalid_argument("Handle " + std::to_string(h) +
                                  " was not created or has been cleared.");
    return it->second;
  }
  void Release(int h) {
    std::lock_guard<std::mutex> l(mu_);
    table_.erase(h);
  }
  void Reset() {
    std::lock_guard<std::mutex> l(mu_);
    table_.clear();
  }

private:
  std::mutex mu_;
  int next_ = 0;
  std::unordered_map<int, std::shared_ptr<HandleRecord>> table_;
};

HandleManager& Handles() {
  static HandleManager* m = new HandleManager();
  return *m;
}

StatusCallback MakeCallback(std::shared_ptr<HandleRecord> rec) {
  return [rec](const Completion& c) {
    std::lock_guard<std::mutex> l(rec->mu);
    if (!c.status.ok() && rec->status.ok()) rec->status = c.status;
    if (c.done_event) rec->done_event = c.done_event;
    if (--rec->pending <= 0) rec->cv.notify_all();
  };
}

// ---- op context -----------------------------------------------------------

class TorchOpContext : public OpContext {
public:
  // index >= 0: the output takes that position of the handle's output list
  // (grouped ops, whose members may complete in any order).
  TorchOpContext(std::shared_ptr<HandleRecord> rec, at::TensorOptions options,
                 int device, int index = -1)
      : rec_(std::move(rec)), options_(options), device_(device), index_(index) {}

  Status AllocateOutput(const TensorShape& shape, void* stream,
                        void** data) override {
    try {
      at::Tensor out;
      if (device_ != CPU_DEVICE_ID) {
        c10::cuda::CUDAGuard guard(device_);
        out = at::empty(shape.to_vector(), options_);
      } else {
        out = at::empty(shape.to_vector(), options_);
      }
      *data = out.data_ptr();
      std::lock_guard<std::mutex> l(rec_->mu);
      if (index_ >= 0 && index_ < static_cast<int>(rec_->outputs.size()))
        rec_->outputs[index_] = std::move(out);
      else
        rec_->outputs.push_back(std::move(out));
      return Status::OK();
    } catch (const std::exception& e) {
      return Status::UnknownError(std::string("output allocation failed: ") +
                                  e.what());
    }
  }
  void SetReceivedSplits(const std::vector<int32_t>& splits) override {
    std::lock_guard<std::mutex> l(rec_->mu);
    rec_->received_splits = splits;
    rec_->has_splits = true;
  }

private:
  std::shared_ptr<HandleRecord> rec_;
  at::TensorOptions options_;
  int device_;
  int index_;
};

void ThrowIfError(const Status& s) {
  switch (s.type()) {
  case StatusType::OK:
  case StatusType::IN_PROGRESS:
    return;
  case StatusType::INVALID_ARGUMENT:
    throw std::invalid_argument(s.reason());
  case StatusType::PRECONDITION_ERROR:
    throw std::logic_error(s.reason());
  default:
    throw std::runtime_error(s.reason());
  }
}

std::string NameOrDefault(const std::string& name, const char* op, int handle) {
  if (!name.empty()) return name;
  return std::string(op) + ".noname." + std::to_string(handle);
}

// Element-wise collectives accept any dense layout (e.g. channels_last) as
// long as the output has the same strides; the others need row-major.
void CheckLayout(const at::Tensor& input, const at::Tensor* output,
                 bool dense_ok) {
  bool ok = input.is_contiguous() ||
            (dense_ok && input.is_non_overlapping_and_dense() &&
             (output == nullptr || output->strides() == input.strides()));
  if (!ok)
    throw std::invalid_argument(
        "Horovod collectives need contiguous tensors; call .contiguous().");
}

TensorTableEntry MakeEntry(const at::Tensor& input, const at::Tensor* output,
                           const std::shared_ptr<HandleRecord>& rec,
                           bool dense_ok = false) {
  CheckLayout(input, output, dense_ok);
  TensorTableEntry e;
  e.input = input.data_ptr();
  e.output = output ? output->data_ptr() : nullptr;
  e.shape = TensorShape(input.sizes().vec());
  e.dtype = ToDataType(input.scalar_type());
  e.wire_dtype = e.dtype;
  e.device = DeviceOf(input);
  e.context = std::make_shared<TorchOpContext>(rec, input.options(), e.device);
  if (e.device != CPU_DEVICE_ID)
    e.ready = std::make_shared<TorchReadyEvent>(e.device);
  e.callback = MakeCallback(rec);
  return e;
}

void FailHandle(int handle, const Status& st) {
  Handles().Release(handle);
  ThrowIfError(st);
}

// ---- ops ------------------------------------------------------------------

int AllreduceAsync(const at::Tensor& tensor, const at::Tensor& output,
                   const std::string& name, int op, double prescale,
                   double postscale, int process_set, int wire_dtype) {
  auto rec = std::make_shared<HandleRecord>();
  rec->device = DeviceOf(tensor);
  rec->inputs = {tensor};
  rec->outputs = {output};
  int handle = Handles().Allocate(rec);
  std::vector<TensorTableEntry> entries;
  try {
    entries.push_back(MakeEntry(tensor, &output, rec, /*dense_ok=*/true));
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  entries[0].name = NameOrDefault(name, "allreduce", handle);
  entries[0].wire_dtype =
      wire_dtype >= 0 ? static_cast<DataType>(wire_dtype) : entries[0].dtype;
  Status st = EnqueueTensorAllreduces(entries, static_cast<ReduceOp>(op),
                                      prescale, postscale, process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

int GroupedAllreduceAsync(const std::vector<at::Tensor>& tensors,
                          const std::vector<at::Tensor>& outputs,
                          const std::string& name, int op, double prescale,
                          double postscale, int process_set, int wire_dtype) {
  if (tensors.size() != outputs.size())
    throw std::invalid_argument("grouped_allreduce: tensors/outputs mismatch");
  auto rec = std::make_shared<HandleRecord>();
  rec->pending = static_cast<int>(tensors.size());
  rec->device = tensors.empty() ? CPU_DEVICE_ID : DeviceOf(tensors[0]);
  rec->inputs = tensors;
  rec->outputs = outputs;
  int handle = Handles().Allocate(rec);
  if (tensors.empty()) {
    rec->pending = 0;
    return handle;
  }
  std::string base = NameOrDefault(name, "grouped_allreduce", handle);
  std::vector<TensorTableEntry> entries;
  try {
    // One ready event serves the whole group (same stream, recorded after
    // the last producer).
    std::shared_ptr<ReadyEvent> shared_ready;
    for (size_t i = 0; i < tensors.size(); ++i) {
      if (DeviceOf(tensors[i]) != rec->device)
        throw std::invalid_argument(
            "grouped_allreduce: all tensors must be on the same device");
      TensorTableEntry e;
      CheckLayout(tensors[i], &outputs[i], /*dense_ok=*/true);
      e.input = tensors[i].data_ptr();
      e.output = outputs[i].data_ptr();
      e.shape = TensorShape(tensors[i].sizes().vec());
      e.dtype = ToDataType(tensors[i].scalar_type());
      e.wire_dtype = wire_dtype >= 0 ? static_cast<DataType>(wire_dtype) : e.dtype;
      e.device = rec->device;
      if (e.device != CPU_DEVICE_ID) {
        if (!shared_ready)
          shared_ready = std::make_shared<TorchReadyEvent>(e.device);
        e.ready = shared_ready;
      }
      e.callback = MakeCallback(rec);
      e.name = base + "_" + std::to_string(i + 1) + "of" +
               std::to_string(tensors.size());
      entries.push_back(std::move(e));
    }
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  Status st = EnqueueTensorAllreduces(entries, static_cast<ReduceOp>(op),
                                      prescale, postscale, process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

int AllgatherAsync(const at::Tensor& tensor, const std::string& name,
                   int process_set) {
  auto rec = std::make_shared<HandleRecord>();
  rec->device = DeviceOf(tensor);
  rec->inputs = {tensor};
  int handle = Handles().Allocate(rec);
  TensorTableEntry e;
  try {
    e = MakeEntry(tensor, nullptr, rec);
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  e.name = NameOrDefault(name, "allgather", handle);
  Status st = EnqueueTensorAllgather(std::move(e), process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

int BroadcastAsync(const at::Tensor& tensor, const at::Tensor& output,
                   int root_rank, const std::string& name, int process_set) {
  auto rec = std::make_shared<HandleRecord>();
  rec->device = DeviceOf(tensor);
  rec->inputs = {tensor};
  rec->outputs = {output};
  int handle = Handles().Allocate(rec);
  TensorTableEntry e;
  try {
    e = MakeEntry(tensor, &output, rec, /*dense_ok=*/true);
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  e.name = NameOrDefault(name, "broadcast", handle);
  Status st = EnqueueTensorBroadcast(std::move(e), root_rank, process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

int AlltoallAsync(const at::Tensor& tensor, const std::vector<int32_t>& splits,
                  const std::string& name, int process_set) {
  auto rec = std::make_shared<HandleRecord>();
  rec->device = DeviceOf(tensor);
  rec->inputs = {tensor};
  int handle = Handles().Allocate(rec);
  TensorTableEntry e;
  try {
    e = MakeEntry(tensor, nullptr, rec);
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  e.splits = splits;
  e.name = NameOrDefault(name, "alltoall", handle);
  Status st = EnqueueTensorAlltoall(std::move(e), process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

int ReducescatterAsync(const at::Tensor& tensor, const std::string& name,
                       int op, double prescale, double postscale,
                       int process_set) {
  auto rec = std::make_shared<HandleRecord>();
  rec->device = DeviceOf(tensor);
  rec->inputs = {tensor};
  int handle = Handles().Allocate(rec);
  TensorTableEntry e;
  try {
    e = MakeEntry(tensor, nullptr, rec);
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  e.name = NameOrDefault(name, "reducescatter", handle);
  Status st = EnqueueTensorReducescatter(std::move(e), static_cast<ReduceOp>(op),
                                         prescale, postscale, process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

// Grouped allgather / reducescatter: one handle for the list; the outputs
// (allocated by the ops) come back in order.
namespace {
std::vector<TensorTableEntry> GroupEntries(const std::vector<at::Tensor>& tensors,
                                           const std::shared_ptr<HandleRecord>& rec,
                                           const std::string& base, const char* op) {
  std::vector<TensorTableEntry> entries;
  std::shared_ptr<ReadyEvent> shared_ready;
  rec->outputs.resize(tensors.size());
  for (size_t i = 0; i < tensors.size(); ++i) {
    if (DeviceOf(tensors[i]) != rec->device)
      throw std::invalid_argument(std::string(op) +
                                  ": all tensors must be on the same device");
    CheckLayout(tensors[i], nullptr, /*dense_ok=*/false);
    TensorTableEntry e;
    e.input = tensors[i].data_ptr();
    e.shape = TensorShape(tensors[i].sizes().vec());
    e.dtype = ToDataType(tensors[i].scalar_type());
    e.wire_dtype = e.dtype;
    e.device = rec->device;
    e.context = std::make_shared<TorchOpContext>(rec, tensors[i].options(), e.device,
                                                 static_cast<int>(i));
    if (e.device != CPU_DEVICE_ID) {
      if (!shared_ready) shared_ready = std::make_shared<TorchReadyEvent>(e.device);
      e.ready = shared_ready;
    }
    e.callback = MakeCallback(rec);
    e.name = base + "_" + std::to_string(i + 1) + "of" + std::to_string(tensors.size());
    entries.push_back(std::move(e));
  }
  return entries;
}
}  // namespace

int GroupedAllgatherAsync(const std::vector<at::Tensor>& tensors, const std::string& name,
                          int process_set) {
  auto rec = std::make_shared<HandleRecord>();
  rec->pending = static_cast<int>(tensors.size());
  rec->device = tensors.empty() ? CPU_DEVICE_ID : DeviceOf(tensors[0]);
  rec->inputs = tensors;
  int handle = Handles().Allocate(rec);
  if (tensors.empty()) return handle;
  std::vector<TensorTableEntry> entries;
  try {
    entries = GroupEntries(tensors, rec, NameOrDefault(name, "grouped_allgather", handle),
                           "grouped_allgather");
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  Status st = EnqueueTensorAllgathers(entries, process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

int GroupedReducescatterAsync(const std::vector<at::Tensor>& tensors, const std::string& name,
                              int op, double prescale, double postscale, int process_set) {
  auto rec = std::make_shared<HandleRecord>();
  rec->pending = static_cast<int>(tensors.size());
  rec->device = tensors.empty() ? CPU_DEVICE_ID : DeviceOf(tensors[0]);
  rec->inputs = tensors;
  int handle = Handles().Allocate(rec);
  if (tensors.empty()) return handle;
  std::vector<TensorTableEntry> entries;
  try {
    entries = GroupEntries(tensors, rec, NameOrDefault(name, "grouped_reducescatter", handle),
                           "grouped_reducescatter");
  } catch (...) {
    Handles().Release(handle);
    throw;
  }
  Status st = EnqueueTensorReducescatters(entries, static_cast<ReduceOp>(op), prescale,
                                          postscale, process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

int JoinAsync(int process_set) {
  auto rec = std::make_shared<HandleRecord>();
  int handle = Handles().Allocate(rec);
  TensorTableEntry e;
  e.output = &rec->join_result;
  e.callback = MakeCallback(rec);
  Status st = EnqueueJoin(std::move(e), process_set);
  if (!st.ok()) FailHandle(handle, st);
  return handle;
}

bool Poll(int handle) {
  auto rec = Handles().Get(handle);
  std::lock_guard<std::mutex> l(rec->mu);
  return rec->pending <= 0;
}

// Waits until the op was executed (CPU) or launched (GPU, in which case the
// current stream is chained behind it), clears the handle and returns
// (outputs, received_splits or None, join_result).
py::tuple WaitAndClear(int handle) {
  auto rec = Handles().Get(handle);
  {
    py::gil_scoped_release release;
    std::unique_lock<std::mutex> l(rec->mu);
    if (rec->pending > 0) {
      // Tell the background loop that somebody is waiting, so that it
      // negotiates now instead of sleeping out its cycle.
      hvd_waiter_enter();
      rec->cv.wait(l, [&] { return rec->pending <= 0; });
      hvd_waiter_exit();
    }
  }
  Handles().Release(handle);
  ThrowIfError(rec->status);
  if (rec->done_event && rec->device != CPU_DEVICE_ID) {
    c10::cuda::CUDAGuard guard(rec->device);  // see TorchReadyEvent
    auto stream = at::cuda::getCurrentCUDAStream(rec->device);
    cudaStreamWaitEvent(stream.stream(),
                        static_cast<cudaEvent_t>(rec->done_event.get()), 0);
    for (auto& t : rec->outputs)
      if (t.defined() && t.is_cuda())
        c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(),
                                                      stream);
  }
  py::object splits = py::none();
  if (rec->has_splits) splits = py::cast(rec->received_splits);
  return py::make_tuple(rec->outputs, splits, rec->join_result);
}

void Init(int rank, int size, int local_rank, int local_size, int cross_rank,
          int cross_size, const std::vector<std::string>& addrs,
          uint64_t token, const std::vector<std::vector<int>>& process_sets) {
  InitConfig cfg;
  cfg.rank = rank;
  cfg.size = size;
  cfg.local_rank = local_rank;
  cfg.local_size = local_size;
  cfg.cross_rank = cross_rank;
  cfg.cross_size = cross_size;
  cfg.peer_addrs = addrs;
  cfg.token = token;
  cfg.process_sets = process_sets;
  RegisterGpuOps();
  py::gil_scoped_release release;
  hvd_init(cfg);
}

void Shutdown() {
  {
    py::gil_scoped_release release;
    hvd_shutdown();
  }
  Handles().Reset();
}

}  // namespace
}  // namespace hvd

PYBIND11_MODULE(_C, m) {
  using namespace hvd;
  m.doc() = "horovod_b200 native runtime";
  m.def("listen", &hvd_listen);
  m.def("init", &Init);
  m.def("shutdown", &Shutdown);
  m.def("is_initialized", &hvd_is_initialized);
  m.def("has_topology", &hvd_has_topology);
  m.def("rank", &hvd_rank);
  m.def("size", &hvd_size);
  m.def("local_rank", &hvd_local_rank);
  m.def("local_size", &hvd_local_size);
  m.def("cross_rank", &hvd_cross_rank);
  m.def("cross_size", &hvd_cross_size);
  m.def("is_homogeneous", &hvd_is_homogeneous);
  m.def("start_timeline", &hvd_start_timeline);
  m.def("stop_timeline", &hvd_stop_timeline);
  m.def("add_process_set", [](const std::vector<int>& ranks) {
    py::gil_scoped_release release;
    return hvd_add_process_set(ranks);
  });
  m.def("remove_process_set", [](int id) {
    py::gil_scoped_release release;
    hvd_remove_process_set(id);
  });
  m.def("process_set_rank", &hvd_process_set_rank);
  m.def("process_set_size", &hvd_process_set_size);
  m.def("process_set_included", &hvd_process_set_included);
  m.def("process_set_ranks", &hvd_process_set_ranks);
  m.def("process_set_ids", &hvd_process_set_ids);

  m.def("allreduce_async", &AllreduceAsync, py::arg("tensor"), py::arg("output"),
        py::arg("name"), py::arg("op"), py::arg("prescale"), py::arg("postscale"),
        py::arg("process_set"), py::arg("wire_dtype") = -1);
  m.def("grouped_allgather_async", &GroupedAllgatherAsync, py::arg("tensors"),
        py::arg("name") = "", py::arg("process_set") = 0);
  m.def("grouped_reducescatter_async", &GroupedReducescatterAsync, py::arg("tensors"),
        py::arg("name") = "", py::arg("op") = 1, py::arg("prescale") = 1.0,
        py::arg("postscale") = 1.0, py::arg("process_set") = 0);
  m.def("grouped_allreduce_async", &GroupedAllreduceAsync, py::arg("tensors"),
        py::arg("outputs"), py::arg("name"), py::arg("op"), py::arg("prescale"),
        py::arg("postscale"), py::arg("process_set"), py::arg("wire_dtype") = -1);
  m.def("allgather_async", &AllgatherAsync);
  m.def("broadcast_async", &BroadcastAsync);
  m.def("alltoall_async", &AlltoallAsync);
  m.def("reducescatter_async", &ReducescatterAsync);
  m.def("join_async", &JoinAsync);
  m.def("poll", &Poll);
  m.def("wait_and_clear", &WaitAndClear);
  m.def("runtime_params", []() {
    // The knob values in effect right now (the autotuner may have moved them).
    py::dict d;
    if (!hvd_is_initialized()) return d;
    const ParameterManager& pm = hvd_state().parameter_manager;
    d["fusion_threshold_bytes"] = pm.TensorFusionThresholdBytes();
    d["cycle_time_ms"] = pm.CycleTimeMs();
    d["cache_enabled"] = pm.CacheEnabled();
    d["hierarchical_allreduce"] = pm.HierarchicalAllreduce();
    d["hierarchical_allgather"] = pm.HierarchicalAllgather();
    d["autotune"] = pm.IsAutoTuning();
    // Whether the rank layout allows the two-level collectives at all.
    d["hierarchy_usable"] = hvd_state().hierarchy_usable;
    return d;
  }, "Fusion threshold, cycle time and the other tunables as they are in effect now.");

  BindGpuDiagnostics(m);
  BindTesting(m);
  BindModelOps(m);
  BindEmulation(m);
}
