// Interface between the background loop and the code that actually moves
// data. One implementation serves host tensors over the TCP mesh, another
// serves device tensors with the NVLink kernels (or NCCL).
//
// Parity: horovod/common/ops/operation_manager.cc:40-121 and the op base
// classes in horovod/common/ops/collective_operations.h:38-299. There is no
// ordered list of alternative backends here: the device alone decides.
#pragma once

#include <vector>

#include "../common/common.h"
#include "../common/message.h"

namespace hvd {

struct ProcessSet;
struct GlobalState;

class OpExecutor {
public:
  virtual ~OpExecutor() = default;
  // Runs the collective described by `response` on `entries` (in response
  // order). Returns OK when the entries' results are final, IN_PROGRESS when
  // the executor will call entry.Finish() itself later, or an error.
  virtual Status Execute(std::vector<TensorTableEntry>& entries,
                         const Response& response, ProcessSet& ps) = 0;
  // Called on the background thread before the mesh goes away.
  virtual void Shutdown() {}
};

}  // namespace hvd
