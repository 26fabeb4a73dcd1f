// Python access to device-side diagnostics and raw kernel entry points.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../kernels/kernels.h"
#include "../ops/gpu_ops.h"

namespace py = pybind11;

namespace hvd {

void BindGpuDiagnostics(py::module_& m) {
  m.def("gpu_backend", &GpuBackendDescription);
  m.def("kernel_launch_count", &kern::KernelLaunchCount,
        "Kernels of this library launched so far in this process.");
}

}  // namespace hvd
