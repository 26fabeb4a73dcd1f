// Everything the background thread owns, in one place.
//
// Parity: horovod/common/global_state.h:39-126.
#pragma once

#include <atomic>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../ops/op_executor.h"
#include "../transport/mesh.h"
#include "parameter_manager.h"
#include "process_set.h"
#include "timeline.h"

namespace hvd {

// Rank layout and rendezvous result handed to init by the Python layer.
struct InitConfig {
  int rank = 0, size = 1;
  int local_rank = 0, local_size = 1;
  int cross_rank = 0, cross_size = 1;
  // peer_addrs[i] = "host:port" rank i listens on (from hvd_listen()).
  std::vector<std::string> peer_addrs;
  uint64_t token = 0;
  std::vector<std::vector<int>> process_sets;  // extra sets registered at init
};

struct GlobalState {
  std::atomic<bool> initialization_done{false};
  std::atomic<bool> init_failed{false};
  std::string init_error;
  std::atomic<bool> shut_down{false};       // asked to stop
  std::atomic<bool> loop_exited{true};      // background thread is gone
  std::thread background_thread;

  InitConfig config;
  bool is_homogeneous = true;
  std::vector<int> local_sizes;  // local_size of every rank
  // Ranks that share this rank's host (its cross_rank), and ranks with this
  // rank's local_rank on the other hosts: the two levels of the hierarchical
  // collectives. `hierarchy_usable` says that every host runs the same number
  // of ranks and that global ranks are numbered host by host, which those
  // algorithms rely on.
  Comm local_comm, cross_comm;
  bool hierarchy_usable = false;

  TcpMesh mesh;
  Timeline timeline;
  bool timeline_mark_cycles = false;
  ParameterManager parameter_manager;
  ProcessSetTable process_sets;

  std::unique_ptr<OpExecutor> cpu_ops;
  std::unique_ptr<OpExecutor> gpu_ops;  // null when built/run without CUDA

  bool elastic_enabled = false;
  bool dynamic_process_sets = false;

  // Error that took the loop down (reported by later API calls).
  std::mutex error_mu;
  std::string fatal_error;

  // Requests from API threads handled on the background thread.
  std::mutex ctl_mu;
  std::condition_variable ctl_cv;
  // Threads blocked in synchronize() on an op that has not been executed yet.
  // While there are any, the background loop does not sleep out its cycle
  // time: what the caller waits for is negotiated at once (HOROVOD_FLUSH_ON_WAIT).
  std::atomic<int> sync_waiters{0};
  std::mutex wake_mu;
  std::condition_variable wake_cv;
  bool flush_on_wait = true;
  std::string pending_timeline_file;   // non-empty: start; with stop flag: stop
  bool pending_timeline_start = false;
  bool pending_timeline_stop = false;
  bool pending_timeline_mark_cycles = false;
  struct PendingSetChange {
    bool add;
    std::vector<int> ranks;  // add
    int32_t id;              // remove / result of add
    bool done = false;
    std::string error;
  };
  std::vector<std::shared_ptr<PendingSetChange>> pending_set_changes;
};

}  // namespace hvd
