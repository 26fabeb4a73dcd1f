// Device-side executor: runs negotiated collectives on CUDA tensors with the
// NVLink kernels over symmetric memory, or with NCCL when that backend is
// selected or symmetric memory cannot be set up.
//
// Parity: horovod/common/ops/gpu_operations.cc:30-386 (stream/event
// discipline, fusion pack/unpack, finalizer) and nccl_operations.cc:65-727.
#pragma once

#include <memory>
#include <string>

#include "op_executor.h"

namespace hvd {

// Installs the GPU executor factory into the runtime (idempotent). Must be
// called before hvd_init() for CUDA tensors to be accepted.
void RegisterGpuOps();

// Human-readable description of the device backend of the running job
// ("symm nvls=1 peers=8 ...", "nccl", "none").
std::string GpuBackendDescription();

}  // namespace hvd
