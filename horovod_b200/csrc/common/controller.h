// Per-process-set negotiator. Every cycle it turns the requests this rank
// enqueued into the ordered list of responses that ALL ranks of the set will
// execute identically. Steady state is one bit-vector allreduce (response
// cache fast path); anything new goes through the set's coordinator (set
// rank 0), which checks that every rank asked for the same thing and answers
// with either an executable response or an ERROR response naming the
// mismatch, so a disagreement raises on every rank instead of hanging.
//
// Parity: horovod/common/controller.h:37-226, controller.cc:73-984. Unlike
// the reference there is no transport subclass (MPI/Gloo controllers): the
// controller talks to `Comm` directly.
#pragma once

#include <deque>
#include <functional>
#include <string>
#include <unordered_map>
#include <vector>

#include "../transport/mesh.h"
#include "group_table.h"
#include "message.h"
#include "parameter_manager.h"
#include "response_cache.h"
#include "stall_inspector.h"
#include "tensor_queue.h"
#include "timeline.h"

namespace hvd {

struct ControllerOptions {
  int64_t fusion_threshold_bytes = 128 * 1024 * 1024;
  bool disable_group_fusion = false;
  uint32_t cache_capacity = 1024;
  // Ranks per node: the threshold is kept a multiple of
  // local_size * FUSION_ATOMIC_UNIT so per-rank shards stay aligned.
  int local_size = 1;
};

// The fusion policy itself: greedily merges the responses that follow a
// fusable one while they are compatible (same type, devices, dtype, scale
// factors, reduce op, wire type; same root for broadcasts) and the total stays
// within `threshold`; responses that do not fit are looked past as long as
// what was skipped would still have fitted (they keep their order).
// `bytes_of` is the fused size of one response.
void FuseResponseQueue(std::deque<Response>& responses, int64_t threshold,
                       const std::function<int64_t(const Response&)>& bytes_of,
                       ResponseList& out);

class Controller {
public:
  Controller(Comm* comm, TensorQueue& queue, ResponseCache& cache,
             GroupTable& groups, Timeline& timeline,
             ParameterManager& params)
      : comm_(comm), queue_(queue), cache_(cache), groups_(groups),
        timeline_(timeline), params_(params), stall_(cache) {}

  int rank() const { return comm_->rank(); }
  int size() const { return comm_->size(); }
  bool is_coordinator() const { return comm_->rank() == 0; }
  StallInspector& stall_inspector() { return stall_; }
  ControllerOptions& options() { return opts_; }

  // Join bookkeeping for this process set (mirrors ProcessSet::joined*).
  struct JoinState {
    bool joined = false;      // this rank called join()
    int joined_size = 0;      // coordinator: ranks that joined so far
    int last_joined_rank = -1;
  };

  // One negotiation round. May throw TransportError.
  ResponseList ComputeResponseList(bool shutdown_requested, JoinState& join);

  // Broadcasts the coordinator's autotuned parameters to the set.
  void SynchronizeParameters();

  int64_t TensorFusionThresholdBytes() const;

private:
  // Coordinator bookkeeping: requests seen so far for each tensor name.
  bool IncrementTensorCount(const Request& msg, int joined_size);
  Response ConstructResponse(const std::string& name, int joined_size);
  void FuseResponses(std::deque<Response>& responses, ResponseList& out);
  void CoordinateCacheAndState(CacheCoordinator& cc);
  int64_t ResponseBytes(const Response& r) const;

  Comm* comm_;
  TensorQueue& queue_;
  ResponseCache& cache_;
  GroupTable& groups_;
  Timeline& timeline_;
  ParameterManager& params_;
  StallInspector stall_;
  ControllerOptions opts_;
  std::unordered_map<std::string, std::vector<Request>> message_table_;
};

}  // namespace hvd
