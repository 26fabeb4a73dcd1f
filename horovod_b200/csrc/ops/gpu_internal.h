// Private declarations shared by the files that implement the device
// executor (gpu_ops.cc: lifecycle and dispatch; gpu_symm_ops.cc: the NVLink
// kernel paths; nccl_ops.cc: the NCCL path).
#pragma once

#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "../common/global_state.h"
#include "../common/thread_pool.h"
#include "../kernels/kernels.h"
#include "../symm/symm_arena.h"
#include "op_executor.h"
#include "exchange_plan.h"

namespace hvd {

#define HVD_CUDA(call)                                                        \
  do {                                                                        \
    cudaError_t e_ = (call);                                                  \
    if (e_ != cudaSuccess)                                                    \
      throw std::runtime_error(std::string(#call) + " failed: " +             \
                               cudaGetErrorString(e_));                       \
  } while (0)

// Pool of completion events; an event returns to the pool when the last
// holder (a handle record in the binding) lets go of it.
class DoneEventPool : public std::enable_shared_from_this<DoneEventPool> {
public:
  std::shared_ptr<void> Get();

private:
  std::mutex mu_;
  std::vector<cudaEvent_t> free_;
};

// Ring of host-pinned / device buffer pairs used to hand per-launch
// descriptors (tensor lists, exchange plans) to kernels: fill the host half,
// one async copy, kernel reads the device half. A slot is reused only after
// the kernel that read it has finished.
class DescriptorRing {
public:
  struct Slot {
    int index = 0;
    char* host = nullptr;
    char* dev = nullptr;
    size_t capacity = 0;
    size_t used = 0;
    // Reserves `bytes` (256-byte aligned) and returns host/device addresses.
    template <typename T> T* Alloc(size_t count, T** dev_ptr) {
      size_t bytes = (count * sizeof(T) + 255) & ~size_t(255);
      if (used + bytes > capacity) return nullptr;
      T* h = reinterpret_cast<T*>(host + used);
      *dev_ptr = reinterpret_cast<T*>(dev + used);
      used += bytes;
      return h;
    }
  };
  ~DescriptorRing();
  void Create(size_t slot_bytes, int slots);
  void Destroy();
  Slot Acquire();
  void Commit(Slot& slot, cudaStream_t stream);
  void Release(const Slot& slot, cudaStream_t stream);
  size_t slot_bytes() const { return slot_bytes_; }

private:
  struct SlotState {
    cudaEvent_t done = nullptr;
    bool used = false;
  };
  size_t slot_bytes_ = 0;
  char* host_ = nullptr;
  char* dev_ = nullptr;
  std::vector<SlotState> slots_;
  int next_ = 0;
};

// What a process set needs to run kernels over the arena: the subset of
// peer pointers in set-rank order, its flag region and its epoch counter.
struct SymmSet {
  int rank = 0;
  int world = 1;
  bool nvls = false;  // multicast usable (set covers the whole arena)
  char* local = nullptr;
  char* peers[SYMM_MAX_RANKS] = {};
  char* mc = nullptr;
  uint32_t* flags_local = nullptr;
  uint32_t* flags_peers[SYMM_MAX_RANKS] = {};
  uint32_t epoch = 0;
  size_t data_bytes = 0;  // general staging capacity
  // Global set only: two small regions behind the general staging area that
  // one-shot allreduces alternate between, which lets them drop their
  // trailing barrier (a region is rewritten only two launches later, after
  // every peer has passed the barrier of the launch in between).
  int64_t oneshot_off[2] = {0, 0};
  int64_t oneshot_bytes = 0;
  uint32_t oneshot_count = 0;
  // Global set only: two regions that the exchange kernel (allgather,
  // broadcast, alltoall) alternates between. A rank stages outbound data in
  // its own region; reuse is guarded by per-launch credits (see
  // kern::ExchangePlan), so these launches need no trailing barrier. Other
  // sets stage in the general area and end with a barrier.
  int64_t xchg_off[2] = {0, 0};
  int64_t xchg_bytes = 0;
  uint32_t xchg_seq = 0;  // exchange launches so far (credit numbers)
};

class NcclOps;

class GpuOps : public OpExecutor {
public:
  // `slot`: which of this process's devices (in order of first use) this
  // executor serves; see MultiDeviceGpuOps.
  // `lane` of `lanes`: which of the communication streams of that device
  // (HOROVOD_NUM_NCCL_STREAMS) this executor is.
  explicit GpuOps(GlobalState& s, int slot = 0, int lane = 0, int lanes = 1);
  ~GpuOps() override;

  Status Execute(std::vector<TensorTableEntry>& entries,
                 const Response& response, ProcessSet& ps) override;
  void Shutdown() override;

  // Segments handed to the exchange kernel (see exchange_plan.h).
  using StageSeg = ExchangeStageSeg;
  using PullSeg = ExchangePullSeg;
  using RoundBlock = ExchangeRoundBlock;

  // Device-time record of one executed response (HOROVOD_GPU_OP_TIMING=1).
  struct OpTiming {
    int type;        // Response::Type
    int64_t bytes;   // payload bytes of the response on this rank
    int tensors;
    float device_us;
    float host_us;   // host time between the two timing events being recorded
  };
  // Waits for the recorded ops to finish and returns (and clears) the list.
  std::vector<OpTiming> DrainTimings();

  // Symmetric heap: memory inside the arena that callers can hold tensors
  // in. Allocation is a bump pointer and must be called with the same sizes
  // in the same order on every rank (the offset is what makes a tensor
  // symmetric). Returns the local address, or nullptr when the arena does
  // not exist or the heap is full. Thread-safe.
  void* SymmHeapAlloc(size_t bytes, int64_t* offset);
  // Offset from the arena base if [p, p+bytes) lies inside the local heap.
  bool InSymmHeap(const void* p, int64_t bytes, int64_t* offset) const;
  int64_t symm_heap_bytes() const { return heap_bytes_; }
  int64_t symm_heap_used() const { return heap_used_.load(); }
  int device() const { return device_; }
  const unsigned long long* kernel_trace() const { return trace_host_; }

  // Timeline activities of device work. With the timeline on, the start and
  // the end of a phase are CUDA events recorded on the communication stream;
  // after the op has finished, the finalizer thread turns them into time
  // stamps (event time relative to a calibration event whose host time is
  // known) and replays them into the timeline, so the trace shows when the
  // GPU went through each phase, not when the host queued it.
  // Parity: horovod/common/ops/gpu_operations.h:69-129 (event queue replayed
  // by the finalizer), horovod/common/ops/cuda_operations.cc:102-148.
  void ActStart(const std::vector<TensorTableEntry>& entries, const char* activity);
  void ActEnd(const std::vector<TensorTableEntry>& entries);
  void ActStart(const std::string& tensor, const char* activity);
  void ActEnd(const std::string& tensor);

  // Used by the NCCL path.
  cudaStream_t stream() const { return stream_; }
  DescriptorRing& ring() { return ring_; }
  GlobalState& state() { return state_; }
  void WaitForInputs(const std::vector<TensorTableEntry>& entries);
  Status Complete(std::vector<TensorTableEntry>& entries);

private:
  void EnsureDevice(int device);
  void EnsureArena(ProcessSet& ps);
  SymmSet* GetSymmSet(ProcessSet& ps);
  kern::SymmCtx MakeCtx(SymmSet& set, uint32_t epochs, int64_t staging_off = 0,
                        bool skip_end_barrier = false);
  Status CheckKernelStatus();
  int PickCtas(int64_t bytes) const;
  kern::Algo PickAlgo(const SymmSet& set, DataType wire, int64_t bytes) const;

  Status SymmAllreduce(std::vector<TensorTableEntry>& entries,
                       const Response& response, SymmSet& set, bool adasum);
  Status SymmBroadcast(std::vector<TensorTableEntry>& entries, SymmSet& set);
  Status GroupedReducescatterPush(std::vector<TensorTableEntry>& entries, SymmSet& set,
                                  bool* done);
  Status SymmAllgather(std::vector<TensorTableEntry>& entries,
                       const Response& response, SymmSet& set);
  Status SymmAlltoall(std::vector<TensorTableEntry>& entries, const Response& response,
                      ProcessSet& ps, SymmSet& set);
  Status SymmReducescatter(std::vector<TensorTableEntry>& entries,
                           SymmSet& set);
  // Zero-copy path for tensors living in the symmetric heap. Returns false
  // (and launches nothing) when the entries do not qualify.
  bool TryInplaceAllreduce(std::vector<TensorTableEntry>& entries,
                           const Response& response, SymmSet& set, Status* status);
  // One exchange-kernel launch for the given segment lists.
  void LaunchExchangeSegments(const std::vector<StageSeg>& stage,
                              const std::vector<PullSeg>& pull, SymmSet& set,
                              int64_t round_bytes, const std::vector<RoundBlock>& round,
                              bool copy_engine = false);
  void LaunchExchangeKernel(const std::vector<StageSeg>& stage,
                            const std::vector<PullSeg>& pull, SymmSet& set,
                            int64_t round_bytes, const std::vector<RoundBlock>& round,
                            bool post_credit);
  // Whether an exchange of `total_bytes` writes straight into the receivers'
  // regions (small messages) instead of staging locally.
  bool ExchangePushes(const SymmSet& set, int64_t total_bytes) const;
  // Whether an exchange of `total_bytes` in remote blocks of at least
  // `smallest` bytes each moves its data across NVLink with copy-engine
  // copies (stage locally, barrier, one peer copy per block).
  bool ExchangeUsesCopyEngine(const SymmSet& set, int64_t total_bytes, int64_t smallest,
                              size_t remote_blocks, bool allgather) const;

  GlobalState& state_;
  int slot_ = 0;
  int lane_ = 0, lanes_ = 1;
  std::shared_ptr<DoneEventPool> events_;
  std::string backend_pref_;
  bool async_completion_ = true;
  bool want_nvls_ = true;
  unsigned long long timeout_ns_ = 0;
  int64_t oneshot_max_ = 0, nvls_min_ = 0;
  int forced_ctas_ = 0;
  bool inline_descriptors_ = true;
  std::string forced_algo_;
  int device_ = -1;
  cudaStream_t stream_ = nullptr;
  ThreadPool finalizer_;
  DescriptorRing ring_;
  SymmArena arena_;
  bool arena_tried_ = false;
  int64_t heap_off_ = 0;     // start of the symmetric heap inside the arena
  int64_t heap_bytes_ = 0;
  std::atomic<int64_t> heap_used_{0};
  char* heap_base_ = nullptr;  // local address of heap_off_
  kern::KernelStatus* status_host_ = nullptr;  // mapped pinned memory
  int* status_dev_ = nullptr;
  unsigned long long* tile_counter_ = nullptr;  // device word, see kern::TileSchedule
  unsigned long long tile_base_ = 0;
  int64_t dynamic_min_bytes_ = 0;
  int64_t exchange_chunk_bytes_ = 256 << 10;  // HOROVOD_EXCHANGE_CHUNK_KB
  int64_t exchange_push_max_ = 1 << 20;       // HOROVOD_EXCHANGE_PUSH_MAX_BYTES
  int64_t exchange_ce_min_ = -1;              // HOROVOD_EXCHANGE_COPY_ENGINE_MIN_BYTES (-1 = by op and size)
  int64_t allreduce_subchunk_bytes_ = 64 << 10;  // HOROVOD_ALLREDUCE_SUBCHUNK_KB, 0 = off
  int64_t allreduce_pipeline_min_ = 8 << 20;     // HOROVOD_ALLREDUCE_PIPELINE_MIN_BYTES
  unsigned long long* xchg_done_counter_ = nullptr;  // device word, see kern::ExchangeSync
  unsigned long long xchg_done_base_ = 0;
  unsigned long long* trace_host_ = nullptr;  // mapped pinned, HOROVOD_KERNEL_TRACE=1
  unsigned long long* trace_dev_ = nullptr;
  std::map<int32_t, std::unique_ptr<SymmSet>> sets_;
  std::unique_ptr<NcclOps> nccl_;
  bool shut_down_ = false;

  struct PendingTiming {
    cudaEvent_t t0, t1;
    int type;
    int64_t bytes;
    int tensors;
    double host_t0;
    float host_us;
  };
  // Closes the timing record of the response being executed: called by
  // Complete() right after the last launch, before callbacks run.
  void CloseTiming();
  PendingTiming* open_timing_ = nullptr;
  struct ActivityMark {
    std::vector<std::string> tensors;
    std::string activity;  // empty: the activity ends here
    cudaEvent_t event;
  };
  void PushMark(std::vector<std::string> tensors, const char* activity);
  cudaEvent_t TimedEvent();
  // Host time (NowMicros clock) at which `ev` completed on the device.
  int64_t EventHostMicros(cudaEvent_t ev);
  void Calibrate();
  std::vector<ActivityMark> marks_;           // of the op being executed
  std::mutex timed_mu_;
  std::vector<cudaEvent_t> timed_events_;     // free list (timing enabled)
  cudaEvent_t calib_event_ = nullptr;
  int64_t calib_host_us_ = 0;

  bool timing_ = false;
  std::mutex timing_mu_;
  std::vector<PendingTiming> pending_timings_;
  std::vector<cudaEvent_t> timing_events_;  // free list
};

// Routes every response to the executor of the device its tensors live on.
class MultiDeviceGpuOps : public OpExecutor {
public:
  explicit MultiDeviceGpuOps(GlobalState& s);
  Status Execute(std::vector<TensorTableEntry>& entries, const Response& response,
                 ProcessSet& ps) override;
  void Shutdown() override;

private:
  static constexpr size_t kMaxDevices = 8;
  static constexpr int kMaxStreams = 4;
  GlobalState& state_;
  int num_streams_ = 1;       // HOROVOD_NUM_NCCL_STREAMS
  size_t next_lane_ = 0;
  std::vector<int> devices_;  // device ordinal behind each row of executors_
  // executors_[device slot][lane]: one executor, with its own stream, arena,
  // flag words, NCCL communicators and finalizer thread, per device and
  // communication stream
  // (horovod/common/global_state.h:92-95, operations.cc:436-449).
  std::vector<std::vector<std::unique_ptr<GpuOps>>> executors_;
};

// Timings of every executor of the process (HOROVOD_GPU_OP_TIMING=1).
std::vector<GpuOps::OpTiming> DrainAllGpuTimings();
// Device responses executed so far by the symmetric-memory kernels and by
// the NCCL path (all executors of the process).
void GpuResponsePathCounts(unsigned long long* symm, unsigned long long* nccl);

// The executor of the running job (null when there is none); used by the
// diagnostics binding.
GpuOps* CurrentGpuOps();

// Published for diagnostics.
void SetGpuBackendDescription(const std::string& s);

}  // namespace hvd
