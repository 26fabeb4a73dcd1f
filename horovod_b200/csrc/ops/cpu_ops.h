// Collectives on host tensors, carried by the TCP mesh. This is the whole
// data path of a CPU-only job and the reference semantics every GPU kernel
// is tested against.
//
// Parity: horovod/common/ops/gloo_operations.cc:32-354 and
// mpi_operations.cc:26-453 (allreduce with fusion and scaling, allgatherv,
// broadcast, alltoallv), horovod/common/ops/adasum/adasum.h:194-435 and
// adasum_mpi_operations.cc:30-100 (Adasum). Reducescatter is an extension.
#pragma once

#include <memory>

#include "op_executor.h"

namespace hvd {

std::unique_ptr<OpExecutor> MakeCpuOps(GlobalState& state);

// Adasum of one rank's fused buffer with all other ranks of `comm`
// (power-of-two size), in place. `counts[i]` is the element count of tensor i
// laid out back to back (each start aligned as in the fused buffer via
// `offsets`). Exposed for tests.
class Comm;
void AdasumCPU(Comm& comm, void* buffer, DataType dtype,
               const std::vector<int64_t>& offsets,
               const std::vector<int64_t>& counts, int64_t total_elements);

// Pairwise Adasum combine of two equally long vectors, the closed form used
// at every level: a <- (1 - dot/(2|a|^2)) a + (1 - dot/(2|b|^2)) b.
// Exposed as the oracle for the device kernel tests.
void AdasumCombineReference(const double* a, const double* b, double* out,
                            int64_t n);

}  // namespace hvd
