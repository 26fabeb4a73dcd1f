// A process set is a subset of ranks with its own queue, cache, group table
// and controller, so collectives on different subsets negotiate
// independently. Id 0 is always the global set. Sets can be added/removed at
// run time once every rank has asked for the same change.
//
// Parity: horovod/common/process_set.h:26-173, process_set.cc:38-402.
#pragma once

#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "controller.h"

namespace hvd {

struct ProcessSet {
  ProcessSet(int32_t id_, TcpMesh* mesh, std::vector<int> ranks,
             Timeline& timeline, ParameterManager& params)
      : id(id_), comm(mesh, std::move(ranks)),
        controller(&comm, tensor_queue, response_cache, group_table, timeline,
                   params) {}

  bool IsCurrentProcessIncluded() const { return comm.contains_me(); }
  const std::vector<int>& ranks() const { return comm.global_ranks(); }

  int32_t id;
  Comm comm;
  TensorQueue tensor_queue;
  ResponseCache response_cache;
  GroupTable group_table;
  Controller controller;
  Controller::JoinState join;
};

class ProcessSetTable {
public:
  // Creates set 0 over all mesh ranks.
  void Initialize(TcpMesh* mesh, Timeline* timeline, ParameterManager* params,
                  const ControllerOptions& opts, bool stall_check,
                  int stall_warn_s, int stall_shutdown_s);
  void Clear();

  // Registers a set on this process (called with identical arguments on all
  // ranks, from the background thread). Returns the id; an existing set with
  // the same ranks returns its id.
  int32_t RegisterProcessSet(std::vector<int> ranks);
  void DeregisterProcessSet(int32_t id);

  bool Contains(int32_t id) const;
  ProcessSet& Get(int32_t id);
  std::vector<int32_t> Ids() const;
  // Id of the set with exactly these ranks, or -1.
  int32_t FindId(const std::vector<int>& ranks) const;

private:
  mutable std::recursive_mutex mu_;
  TcpMesh* mesh_ = nullptr;
  Timeline* timeline_ = nullptr;
  ParameterManager* params_ = nullptr;
  ControllerOptions opts_;
  bool stall_check_ = true;
  int stall_warn_s_ = 60, stall_shutdown_s_ = 0;
  std::map<int32_t, std::unique_ptr<ProcessSet>> sets_;
  int32_t next_id_ = 0;
};

}  // namespace hvd
