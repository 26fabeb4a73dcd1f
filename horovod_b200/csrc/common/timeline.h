// Chrome-trace ("chrome://tracing" / Perfetto JSON) timeline of every
// collective: negotiation, queueing, and the activities inside each op.
// Each tensor is shown as its own "process"; events are handed to a writer
// thread so the background loop never blocks on file IO. Can be started and
// stopped while the job runs.
//
// Parity: horovod/common/timeline.h:84-188, timeline.cc:38-678. The
// hand-off queue here is a mutex-guarded vector swapped out by the writer
// (the reference uses a bounded lock-free queue).
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "message.h"

namespace hvd {

// Activity names shown inside an op (same vocabulary as the reference's
// horovod/common/common.h:73-105 where the phase exists in both designs).
#define HVD_ACT_WAIT_FOR_DATA "WAIT_FOR_DATA"
#define HVD_ACT_WAIT_FOR_OTHER_TENSOR_DATA "WAIT_FOR_OTHER_TENSOR_DATA"
#define HVD_ACT_QUEUE "QUEUE"
#define HVD_ACT_MEMCPY_IN_FUSION_BUFFER "MEMCPY_IN_FUSION_BUFFER"
#define HVD_ACT_MEMCPY_OUT_FUSION_BUFFER "MEMCPY_OUT_FUSION_BUFFER"
#define HVD_ACT_ALLOCATE_OUTPUT "ALLOCATE_OUTPUT"
#define HVD_ACT_FUSED_KERNEL "FUSED_NVLINK_KERNEL"
#define HVD_ACT_NCCL_ALLREDUCE "NCCL_ALLREDUCE"
#define HVD_ACT_NCCL_ALLGATHER "NCCL_ALLGATHER"
#define HVD_ACT_NCCL_BCAST "NCCL_BCAST"
#define HVD_ACT_NCCL_ALLTOALL "NCCL_ALLTOALL"
#define HVD_ACT_NCCL_REDUCESCATTER "NCCL_REDUCESCATTER"
#define HVD_ACT_CPU_ALLREDUCE "CPU_ALLREDUCE"
#define HVD_ACT_CPU_ALLGATHER "CPU_ALLGATHER"
#define HVD_ACT_CPU_BCAST "CPU_BCAST"
#define HVD_ACT_CPU_ALLTOALL "CPU_ALLTOALL"
#define HVD_ACT_CPU_REDUCESCATTER "CPU_REDUCESCATTER"
#define HVD_ACT_CPU_ADASUM "CPU_ADASUM"
#define HVD_ACT_INIT_FUSION_BUFFER "INIT_FUSION_BUFFER"

class Timeline {
public:
  Timeline() = default;
  ~Timeline() { Shutdown(); }

  // Opens `file` and starts the writer thread. Safe to call again after
  // Shutdown().
  void Initialize(const std::string& file, bool mark_cycles);
  void Shutdown();
  bool Initialized() const { return active_.load(std::memory_order_acquire); }

  void NegotiateStart(const std::string& tensor, Request::Type type);
  void NegotiateRankReady(const std::string& tensor, int rank);
  void NegotiateEnd(const std::string& tensor);
  void Start(const std::string& tensor, Response::Type type,
             int64_t size_bytes = 0);
  void ActivityStart(const std::string& tensor, const std::string& activity);
  void ActivityEnd(const std::string& tensor);
  void ActivityStartAll(const std::vector<TensorTableEntry>& entries,
                        const std::string& activity);
  void ActivityEndAll(const std::vector<TensorTableEntry>& entries);
  void End(const std::string& tensor);
  void MarkCycleStart();
  // The same three transitions with a time stamp supplied by the caller
  // (microseconds on the NowMicros() clock): the device executor replays the
  // phases of an op with the times at which the GPU actually went through
  // them, taken from CUDA events, after the op has finished.
  void ActivityStartAt(const std::string& tensor, const std::string& activity, int64_t abs_us);
  void ActivityEndAt(const std::string& tensor, int64_t abs_us);
  void EndAt(const std::string& tensor, int64_t abs_us);

private:
  enum class State { UNKNOWN, NEGOTIATING, TOP_LEVEL, ACTIVITY };
  struct Record {
    char phase;            // 'B', 'E', 'X', 'i', 'M'
    std::string tensor;    // empty for cycle markers
    std::string name;
    std::string args;      // raw JSON object body or empty
    int64_t ts_us;
  };
  // abs_us < 0: now.
  void Emit(char phase, const std::string& tensor, const std::string& name,
            const std::string& args = "", int64_t abs_us = -1);
  // Mirrors of the trace in two NVTX domains (ops, and the activities inside
  // them), so that Nsight shows the same structure as the Chrome trace.
  void NvtxPush(bool activity, const std::string& tensor, const std::string& name);
  void NvtxPop(bool activity, const std::string& tensor);
  std::unordered_map<std::string, uint64_t> nvtx_ops_, nvtx_activities_;  // under state_mu_
  void WriterLoop();
  void WriteRecord(const Record& r);

  std::atomic<bool> active_{false};
  bool mark_cycles_ = false;
  int64_t start_us_ = 0;

  std::mutex state_mu_;  // guards states_ (producers on several threads)
  std::unordered_map<std::string, State> states_;

  std::mutex q_mu_;
  std::condition_variable q_cv_;
  std::vector<Record> queue_;
  bool stop_ = false;
  std::thread writer_;

  // Writer-thread state.
  FILE* file_ = nullptr;
  bool first_event_ = true;
  std::unordered_map<std::string, int> tensor_pid_;
};

}  // namespace hvd
