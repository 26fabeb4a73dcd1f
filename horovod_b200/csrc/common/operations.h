// Public C++ surface of the runtime: lifecycle, topology queries, process
// sets, timeline control and the enqueue functions the framework binding
// calls. All enqueue functions return immediately; results arrive through
// each entry's callback.
//
// Parity: horovod/common/operations.h:42-233, operations.cc:257-1742.
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "common.h"
#include "global_state.h"

namespace hvd {

// Step 1 of init: opens this rank's listening socket and returns the
// "host:port" to publish through whatever rendezvous the launcher offers.
std::string hvd_listen(const std::string& advertise_host);
// Step 2: starts the background thread, builds the mesh from
// cfg.peer_addrs and blocks until the runtime is ready. Throws
// std::runtime_error when initialisation fails. Calling it again after
// hvd_shutdown() starts a fresh runtime (elastic reset).
void hvd_init(const InitConfig& cfg);
void hvd_shutdown();
// A thread starts / stops waiting for an op that the background loop has not
// executed yet (see GlobalState::sync_waiters).
void hvd_waiter_enter();
void hvd_waiter_exit();
bool hvd_is_initialized();
bool hvd_has_topology();

int hvd_rank();
int hvd_size();
int hvd_local_rank();
int hvd_local_size();
int hvd_cross_rank();
int hvd_cross_size();
bool hvd_is_homogeneous();

void hvd_start_timeline(const std::string& file, bool mark_cycles);
void hvd_stop_timeline();

// Process sets. add/remove block until every rank asked for the same change
// (dynamic mode) and return the id / throw on error.
int32_t hvd_add_process_set(const std::vector<int>& ranks);
void hvd_remove_process_set(int32_t id);
int hvd_process_set_rank(int32_t id);
int hvd_process_set_size(int32_t id);
bool hvd_process_set_included(int32_t id);
std::vector<int> hvd_process_set_ranks(int32_t id);
std::vector<int32_t> hvd_process_set_ids();

// Installs the factory for the device executor (set by the CUDA part of the
// library when it is linked in).
using GpuOpsFactory = std::function<std::unique_ptr<OpExecutor>(GlobalState&)>;
void hvd_set_gpu_ops_factory(GpuOpsFactory f);

// Enqueue API. Entries must have name, pointers, shape, dtype, device,
// context, ready event and callback filled in.
Status EnqueueTensorAllreduces(std::vector<TensorTableEntry>& entries,
                               ReduceOp op, double prescale, double postscale,
                               int32_t process_set_id);
Status EnqueueTensorAllgather(TensorTableEntry entry, int32_t process_set_id);
// Several tensors as one group: negotiated together and fused into one
// response per dtype (subject to the fusion threshold).
Status EnqueueTensorAllgathers(std::vector<TensorTableEntry>& entries,
                               int32_t process_set_id);
Status EnqueueTensorReducescatters(std::vector<TensorTableEntry>& entries, ReduceOp op,
                                   double prescale, double postscale,
                                   int32_t process_set_id);
Status EnqueueTensorBroadcast(TensorTableEntry entry, int root_rank,
                              int32_t process_set_id);
Status EnqueueTensorAlltoall(TensorTableEntry entry, int32_t process_set_id);
Status EnqueueTensorReducescatter(TensorTableEntry entry, ReduceOp op,
                                  double prescale, double postscale,
                                  int32_t process_set_id);
// entry.output must point at an int32 that receives the last joined rank.
Status EnqueueJoin(TensorTableEntry entry, int32_t process_set_id);

GlobalState& hvd_state();

}  // namespace hvd
