// NCCL data path for device tensors: the measured baseline (it issues the
// same pack -> NCCL call -> unpack sequence per fused response as the
// reference) and the fallback where symmetric memory cannot be used (more
// than one node, more than 8 ranks, reductions other than sum, no peer
// access). The library is opened with dlopen so nothing links against it.
//
// Parity: horovod/common/ops/nccl_operations.cc:65-727.
#pragma once

#include <map>
#include <memory>
#include <vector>

#include "../common/fusion_buffer_manager.h"
#include "nccl_comm_set.h"
#include "op_executor.h"

namespace hvd {

class GpuOps;
class Comm;
struct NcclApi;

class NcclOps {
public:
  explicit NcclOps(GpuOps& gpu);
  ~NcclOps();
  Status Execute(std::vector<TensorTableEntry>& entries,
                 const Response& response, ProcessSet& ps);
  void Shutdown();
  // For the thread that waits for a collective in an elastic job: whether
  // there is anything to watch, and the check itself (nccl_comm_set.h).
  bool HasCommunicators() { return !comms_.empty(); }
  Status CheckAsyncErrors() { return comms_.CheckAsyncErrors(); }

private:
  void* CommFor(ProcessSet& ps);
  // NCCL communicator over the ranks of `comm` (a control-plane communicator
  // this rank belongs to), cached under `key` (negative keys: the host-local
  // and cross-host communicators of the hierarchical allreduce).
  void* CommOver(int32_t key, Comm& comm);
  bool UseHierarchicalAllreduce(const ProcessSet& ps) const;
  void* Fusion(size_t bytes);
  Status Allreduce(std::vector<TensorTableEntry>& entries,
                   const Response& response, void* comm);
  Status Broadcast(std::vector<TensorTableEntry>& entries, void* comm);
  Status Allgather(std::vector<TensorTableEntry>& entries,
                   const Response& response, ProcessSet& ps, void* comm);
  Status Alltoall(std::vector<TensorTableEntry>& entries, const Response& response,
                  ProcessSet& ps,
                  void* comm);
  Status Reducescatter(std::vector<TensorTableEntry>& entries, ProcessSet& ps,
                       void* comm);

  GpuOps& gpu_;
  const NcclApi* api_ = nullptr;
  NcclCommSet comms_;
  FusionBufferManager buffers_;
  bool hierarchical_ = false;  // the allreduce being executed runs in two levels
};

}  // namespace hvd
