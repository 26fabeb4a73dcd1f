// Python access to device-side diagnostics and raw kernel entry points.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../kernels/kernels.h"
#include "../ops/gpu_internal.h"
#include "../ops/gpu_ops.h"
#include "../symm/topology.h"

namespace py = pybind11;

namespace hvd {

void BindGpuDiagnostics(py::module_& m) {
  m.def("gpu_backend", &GpuBackendDescription);
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
  m.def("kernel_launch_count", &kern::KernelLaunchCount,
        "Kernels of this library launched so far in this process.");
}

}  // namespace hvd
