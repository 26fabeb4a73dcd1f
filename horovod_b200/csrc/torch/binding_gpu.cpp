// Python access to device-side diagnostics and raw kernel entry points.
#include <torch/extension.h>

#include <pybind11/stl.h>

#include "../kernels/kernels.h"
#include "../ops/gpu_internal.h"
#include "../ops/gpu_ops.h"
#include "../symm/topology.h"

namespace py = pybind11;

namespace hvd {

void BindGpuDiagnostics(py::module_& m) {
  m.def("gpu_backend", &GpuBackendDescription);
  m.def("symm_empty", [](const std::vector<int64_t>& sizes, py::object dtype) {
    // A tensor inside the symmetric heap (same offset on every rank when all
    // ranks allocate the same sequence). The memory belongs to the arena: it
    // is never freed individually and dies with hvd.shutdown().
    GpuOps* ops = CurrentGpuOps();
    if (ops == nullptr)
      throw std::runtime_error("symmetric memory needs an initialised runtime with a GPU");
    at::ScalarType st = torch::python::detail::py_object_to_dtype(dtype);
    int64_t n = 1;
    for (auto d : sizes) n *= d;
    int64_t off = 0;
    void* p = ops->SymmHeapAlloc(static_cast<size_t>(std::max<int64_t>(n, 1)) *
                                     c10::elementSize(st), &off);
    if (p == nullptr)
      throw std::runtime_error(
          "symmetric heap unavailable or exhausted (backend: " + GpuBackendDescription() +
          "); raise HOROVOD_SYMM_HEAP_MB");
    auto options = at::TensorOptions().dtype(st).device(at::kCUDA, ops->device());
    return at::from_blob(p, sizes, [](void*) {}, options);
  });
  m.def("symm_heap_info", []() {
    GpuOps* ops = CurrentGpuOps();
    py::dict d;
    d["bytes"] = ops ? ops->symm_heap_bytes() : 0;
    d["used"] = ops ? ops->symm_heap_used() : 0;
    return d;
  });
  m.def("gpu_topology", []() {
    GpuTopology t = DiscoverTopology();
    py::dict d;
    d["device_count"] = t.device_count;
    d["names"] = t.names;
    d["sm_counts"] = t.sm_counts;
    d["memory_bytes"] = t.memory_bytes;
    d["multicast_supported"] = t.multicast_supported;
    d["nvlink_active_links"] = t.nvlink_active_links;
    d["peer_access"] = t.peer_access;
    d["native_atomics"] = t.native_atomics;
    d["performance_rank"] = t.performance_rank;
    d["all_pairs_peer"] = t.all_pairs_peer;
    d["summary"] = t.Summary();
    return d;
  });
  m.def("gpu_op_stats", []() {
    // (response type, payload bytes, tensors, device microseconds) of every
    // device collective since the last call; needs HOROVOD_GPU_OP_TIMING=1.
    py::list out;
    GpuOps* ops = CurrentGpuOps();
    if (ops == nullptr) return out;
    std::vector<GpuOps::OpTiming> t;
    {
      py::gil_scoped_release release;
      t = ops->DrainTimings();
    }
    for (auto& x : t) out.append(py::make_tuple(x.type, x.bytes, x.tensors, x.device_us));
    return out;
  });
  m.def("kernel_trace", []() {
    // %globaltimer (ns) at the phase boundaries of the last traced allreduce
    // kernel: 0 start, 1 packed, 2 first barrier passed, 3 reduced,
    // 4 second barrier passed, 5 unpacked. Needs HOROVOD_KERNEL_TRACE=1.
    GpuOps* ops = CurrentGpuOps();
    std::vector<unsigned long long> out;
    if (ops != nullptr && ops->kernel_trace() != nullptr)
      out.assign(ops->kernel_trace(), ops->kernel_trace() + kern::KERNEL_TRACE_SLOTS);
    return out;
  });
  m.def("kernel_launch_count", &kern::KernelLaunchCount,
        "Kernels of this library launched so far in this process.");
}

}  // namespace hvd
