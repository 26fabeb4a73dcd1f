#include "gpu_ops.h"

namespace hvd {
void RegisterGpuOps() {}
std::string GpuBackendDescription() { return "none"; }
}  // namespace hvd
