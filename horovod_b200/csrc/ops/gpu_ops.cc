#include "gpu_ops.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstring>

#include "../common/env.h"
#include "../common/logging.h"
#include "../common/operations.h"
#include "gpu_internal.h"
#include "../symm/topology.h"
#include "nccl_ops.h"
#include "host_trace.h"

namespace hvd {

namespace {
std::mutex g_desc_mu;
std::string g_backend_desc = "none";
std::atomic<GpuOps*> g_current{nullptr};
}  // namespace

GpuOps* CurrentGpuOps() { return g_current.load(); }

namespace {
// Responses executed per device data path since the process started:
// [0] symmetric-memory kernels, [1] NCCL.
std::atomic<unsigned long long> g_path_counts[2];
}  // namespace

void GpuResponsePathCounts(unsigned long long* symm, unsigned long long* nccl) {
  *symm = g_path_counts[0].load();
  *nccl = g_path_counts[1].load();
}

namespace {
// Every live executor (one per device and communication stream), for the
// diagnostics that sum over them.
std::mutex& g_registry_mu_ref() {
  static std::mutex mu;
  return mu;
}
std::vector<GpuOps*>& g_registry_ref() {
  static std::vector<GpuOps*> v;
  return v;
}
}  // namespace

void SetGpuBackendDescription(const std::string& s) {
  std::lock_guard<std::mutex> l(g_desc_mu);
  g_backend_desc = s;
}

std::string GpuBackendDescription() {
  std::lock_guard<std::mutex> l(g_desc_mu);
  return g_backend_desc;
}

void RegisterGpuOps() {
  hvd_set_gpu_ops_factory([](GlobalState& s) -> std::unique_ptr<OpExecutor> {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
      cudaGetLastError();
      SetGpuBackendDescription("none");
      return nullptr;
    }
    SetGpuBackendDescription("pending (no device collective has run yet)");
    return std::unique_ptr<OpExecutor>(new MultiDeviceGpuOps(s));
  });
}

// ---------------------------------------------------------------------------
// One GpuOps per device a process hands tensors from. The usual job has one
// GPU per process and therefore one executor; a process that spreads a model
// over several of its GPUs (layers on two devices of one rank, every rank
// alike) gets one executor, with its own stream, arena and flags, per device.
// Executors are numbered in the order their devices first appear: responses
// are executed in the same order on every rank, so "the second device" means
// the same model stage everywhere, whatever the local device ordinals are.
// Parity: test/parallel/test_torch.py:1860-1904 (model parallelism inside a
// rank is tolerated; the reference keeps one NCCL communicator per device
// vector, horovod/common/ops/nccl_operations.h:40-49).

MultiDeviceGpuOps::MultiDeviceGpuOps(GlobalState& s) : state_(s) {
  num_streams_ = static_cast<int>(
      std::min<int64_t>(kMaxStreams, std::max<int64_t>(1, EnvInt(HVD_ENV_NUM_STREAMS, 1))));
}

Status MultiDeviceGpuOps::Execute(std::vector<TensorTableEntry>& entries,
                                  const Response& response, ProcessSet& ps) {
  int device = -1;
  for (auto& e : entries)
    if (e.device != CPU_DEVICE_ID && (e.input || e.output)) device = e.device;
  size_t slot = 0;
  if (device >= 0) {
    for (; slot < devices_.size(); ++slot)
      if (devices_[slot] == device) break;
    if (slot == devices_.size()) {
      if (slot >= kMaxDevices)
        return Status::PreconditionError(
            "This process uses more than " + std::to_string(kMaxDevices) +
            " CUDA devices with Horovod.");
      devices_.push_back(device);
      executors_.emplace_back();
    }
  } else if (executors_.empty()) {
    // A joined rank's stand-in has no device of its own: use the default.
    devices_.push_back(-1);
    executors_.emplace_back();
  }
  slot = std::min(slot, executors_.size() - 1);
  auto& lanes = executors_[slot];
  // Several communication streams: responses take the lanes in turn (every
  // rank executes the same responses in the same order, so all ranks pick the
  // same lane for a response). Tensors in the symmetric heap belong to the
  // first lane, whose arena holds that heap.
  size_t lane = 0;
  if (num_streams_ > 1) {
    lane = next_lane_++ % static_cast<size_t>(num_streams_);
    if (!lanes.empty() && lanes[0] != nullptr)
      for (auto& e : entries)
        if (e.input != nullptr && lanes[0]->InSymmHeap(e.input, 1, nullptr)) lane = 0;
  }
  if (lanes.size() <= lane) lanes.resize(lane + 1);
  if (lanes[lane] == nullptr)
    lanes[lane].reset(new GpuOps(state_, static_cast<int>(slot), static_cast<int>(lane),
                                 num_streams_));
  return lanes[lane]->Execute(entries, response, ps);
}

void MultiDeviceGpuOps::Shutdown() {
  for (auto& lanes : executors_)
    for (auto& e : lanes)
      if (e) e->Shutdown();
}

std::vector<GpuOps::OpTiming> DrainAllGpuTimings() {
  std::vector<GpuOps*> all;
  {
    std::lock_guard<std::mutex> l(g_registry_mu_ref());
    all = g_registry_ref();
  }
  std::vector<GpuOps::OpTiming> out;
  for (GpuOps* ops : all) {
    auto part = ops->DrainTimings();
    out.insert(out.end(), part.begin(), part.end());
  }
  return out;
}

// ---------------------------------------------------------------------------

std::shared_ptr<void> DoneEventPool::Get() {
  cudaEvent_t e = nullptr;
  {
    std::lock_guard<std::mutex> l(mu_);
    if (!free_.empty()) {
      e = free_.back();
      free_.pop_back();
    }
  }
  if (e == nullptr) HVD_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  std::weak_ptr<DoneEventPool> weak = shared_from_this();
  return std::shared_ptr<void>(e, [weak](void* p) {
    if (auto pool = weak.lock()) {
      std::lock_guard<std::mutex> l(pool->mu_);
      pool->free_.push_back(static_cast<cudaEvent_t>(p));
    }
    // Pool gone (shutdown): the event is reclaimed with the context.
  });
}

DescriptorRing::~DescriptorRing() { Destroy(); }

void DescriptorRing::Create(size_t slot_bytes, int slots) {
  slot_bytes_ = slot_bytes;
  slots_.resize(slots);
  HVD_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&host_), slot_bytes * slots,
                         cudaHostAllocDefault));
  HVD_CUDA(cudaMalloc(reinterpret_cast<void**>(&dev_), slot_bytes * slots));
  for (auto& s : slots_) {
    HVD_CUDA(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
    s.used = false;
  }
}

void DescriptorRing::Destroy() {
  for (auto& s : slots_)
    if (s.done) cudaEventDestroy(s.done);
  slots_.clear();
  if (host_) cudaFreeHost(host_);
  if (dev_) cudaFree(dev_);
  host_ = dev_ = nullptr;
}

DescriptorRing::Slot DescriptorRing::Acquire() {
  SlotState& s = slots_[next_];
  if (s.used) HVD_CUDA(cudaEventSynchronize(s.done));
  Slot out;
  out.index = next_;
  out.host = host_ + slot_bytes_ * next_;
  out.dev = dev_ + slot_bytes_ * next_;
  out.capacity = slot_bytes_;
  out.used = 0;
  next_ = (next_ + 1) % static_cast<int>(slots_.size());
  return out;
}

void DescriptorRing::Commit(Slot& slot, cudaStream_t stream) {
  if (slot.used > 0)
    HVD_CUDA(cudaMemcpyAsync(slot.dev, slot.host, slot.used,
                             cudaMemcpyHostToDevice, stream));
}

void DescriptorRing::Release(const Slot& slot, cudaStream_t stream) {
  SlotState& s = slots_[slot.index];
  HVD_CUDA(cudaEventRecord(s.done, stream));
  s.used = true;
}

// ---------------------------------------------------------------------------

GpuOps::GpuOps(GlobalState& s, int slot, int lane, int lanes)
    : state_(s), slot_(slot), lane_(lane), lanes_(std::max(1, lanes)),
      events_(new DoneEventPool()) {
  backend_pref_ = EnvString(HVD_ENV_GPU_BACKEND, "symm");
  async_completion_ = EnvBool(HVD_ENV_ENABLE_ASYNC_COMPLETION, !s.elastic_enabled);
  want_nvls_ = EnvBool(HVD_ENV_SYMM_NVLS, true);
  timeout_ns_ = static_cast<unsigned long long>(
                    EnvInt(HVD_ENV_SPIN_TIMEOUT_MS, 20000)) * 1000000ull;
  oneshot_max_ = EnvInt(HVD_ENV_ONESHOT_MAX, -1);  // -1: by world size
  nvls_min_ = EnvInt(HVD_ENV_NVLS_MIN, 512 * 1024);
  forced_ctas_ = static_cast<int>(EnvInt(HVD_ENV_COMM_CTAS, 0));
  forced_algo_ = EnvString(HVD_ENV_ALGO, "auto");
  timing_ = EnvBool("HOROVOD_GPU_OP_TIMING", false);
  inline_descriptors_ = EnvBool("HOROVOD_INLINE_DESCRIPTORS", true);
  if (slot == 0 && lane == 0 && !EnvBool(HVD_ENV_BATCH_D2D_MEMCOPIES, true))
    HVD_LOG(WARNING) << HVD_ENV_BATCH_D2D_MEMCOPIES
                     << "=0 has no effect: fused tensors are always moved by one kernel per "
                        "response (there is no per-tensor copy path).";
  if (slot == 0 && lane == 0) g_current = this;  // diagnostics and the symmetric heap
  std::lock_guard<std::mutex> l(g_registry_mu_ref());
  g_registry_ref().push_back(this);
}

GpuOps::~GpuOps() { Shutdown(); }

void GpuOps::EnsureDevice(int device) {
  if (device_ == device) return;
  if (device_ >= 0)
    throw std::runtime_error(
        "internal error: device executor for cuda:" + std::to_string(device_) +
        " was handed a tensor on cuda:" + std::to_string(device));
  HVD_CUDA(cudaSetDevice(device));
  int lo = 0, hi = 0;
  HVD_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  HVD_CUDA(cudaStreamCreateWithPriority(&stream_, cudaStreamNonBlocking, hi));
  ring_.Create(1 << 20, 8);
  HVD_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&status_host_),
                         sizeof(kern::KernelStatus), cudaHostAllocMapped));
  std::memset(status_host_, 0, sizeof(kern::KernelStatus));
  HVD_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev_),
                                    status_host_, 0));
  HVD_CUDA(cudaMalloc(reinterpret_cast<void**>(&tile_counter_), sizeof(unsigned long long)));
  HVD_CUDA(cudaMemset(tile_counter_, 0, sizeof(unsigned long long)));
  tile_base_ = 0;
  dynamic_min_bytes_ = EnvInt("HOROVOD_DYNAMIC_TILES_MIN_BYTES", 8 << 20);
  exchange_chunk_bytes_ =
      std::max<int64_t>(64, EnvInt("HOROVOD_EXCHANGE_CHUNK_KB", 256)) << 10;
  exchange_push_max_ = EnvInt("HOROVOD_EXCHANGE_PUSH_MAX_BYTES", 1 << 20);
  exchange_ce_min_ = EnvInt("HOROVOD_EXCHANGE_COPY_ENGINE_MIN_BYTES", -1);
  allreduce_pipeline_min_ = EnvInt("HOROVOD_ALLREDUCE_PIPELINE_MIN_BYTES", 8 << 20);
  allreduce_subchunk_bytes_ =
      std::max<int64_t>(0, EnvInt("HOROVOD_ALLREDUCE_SUBCHUNK_KB", 64)) * 1024 / 256 * 256;
  HVD_CUDA(cudaMalloc(reinterpret_cast<void**>(&xchg_done_counter_), sizeof(unsigned long long)));
  HVD_CUDA(cudaMemset(xchg_done_counter_, 0, sizeof(unsigned long long)));
  xchg_done_base_ = 0;
  if (EnvBool("HOROVOD_KERNEL_TRACE", false)) {
    HVD_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&trace_host_),
                           kern::KERNEL_TRACE_SLOTS * sizeof(unsigned long long),
                           cudaHostAllocMapped));
    std::memset(trace_host_, 0, kern::KERNEL_TRACE_SLOTS * sizeof(unsigned long long));
    HVD_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void**>(&trace_dev_), trace_host_, 0));
  }
  finalizer_.Start(1);
  device_ = device;
}

void GpuOps::EnsureArena(ProcessSet& ps) {
  if (arena_tried_ || ps.id != 0) return;
  arena_tried_ = true;
  const bool one_node = state_.config.local_size == state_.config.size;
  if (backend_pref_ == "nccl" || !one_node ||
      state_.config.size > SYMM_MAX_RANKS) {
    SetGpuBackendDescription("nccl");
    return;
  }
  if (state_.config.rank == 0)
    HVD_LOG(INFO) << "GPU topology: " << DiscoverTopology().Summary();
  size_t mb = static_cast<size_t>(EnvInt(HVD_ENV_SYMM_BUFFER_MB, 1024));
  // The token doubles as socket-name salt: distinct per job, per init and per
  // device executor of this process.
  uint64_t token = (state_.config.token ^ 0x9e3779b97f4a7c15ull) +
                   0x100000001b3ull * static_cast<uint64_t>(slot_ * 16 + lane_);
  // Only the first lane of a device carries the symmetric heap.
  size_t heap_mb = lane_ == 0 ? static_cast<size_t>(EnvInt("HOROVOD_SYMM_HEAP_MB", 4096)) : 0;
  Status st = arena_.Create(ps.comm, device_, (mb + heap_mb) << 20, want_nvls_, token);
  if (!st.ok()) {
    HVD_LOG(WARNING) << st.reason()
                     << " -- device collectives fall back to NCCL.";
    SetGpuBackendDescription("nccl (symmetric memory unavailable: " +
                             st.reason() + ")");
    return;
  }
  const SymmArenaInfo& a = arena_.info();
  heap_off_ = static_cast<int64_t>(mb << 20);
  heap_bytes_ = static_cast<int64_t>(heap_mb << 20);
  heap_used_ = 0;
  heap_base_ = static_cast<char*>(a.local) + heap_off_;
  SetGpuBackendDescription(
      "symm ranks=" + std::to_string(a.world) + " nvls=" +
      std::to_string(a.multicast ? 1 : 0) + " staging_mb=" + std::to_string(mb) +
      " heap_mb=" + std::to_string(heap_mb));
  HVD_LOG(INFO) << "symmetric memory ready: " << GpuBackendDescription();
}

SymmSet* GpuOps::GetSymmSet(ProcessSet& ps) {
  if (!arena_.valid()) return nullptr;
  auto it = sets_.find(ps.id);
  if (it != sets_.end()) return it->second.get();
  if (ps.id >= SYMM_FLAG_SETS) return nullptr;  // no flag region left
  const SymmArenaInfo& a = arena_.info();
  std::unique_ptr<SymmSet> set(new SymmSet());
  const auto& ranks = ps.ranks();  // global == arena ranks on one node
  set->world = static_cast<int>(ranks.size());
  set->rank = ps.comm.rank();
  set->data_bytes = static_cast<size_t>(heap_off_);  // staging part only
  // Room for the two one-shot regions (kept out of the general staging area
  // for every set, so that no other kernel ever writes there).
  const int64_t region = RoundUp(std::max<int64_t>(oneshot_max_, 4 << 20) + 4096, 4096);
  if (static_cast<int64_t>(set->data_bytes) > 4 * region) {
    set->data_bytes = set->data_bytes - 2 * region;
    if (ps.id == 0) {
      set->oneshot_bytes = region;
      set->oneshot_off[0] = static_cast<int64_t>(set->data_bytes);
      set->oneshot_off[1] = static_cast<int64_t>(set->data_bytes) + region;
    }
  }
  // A quarter of what is left for each of the two exchange regions (again
  // carved out for every set, used by the global one).
  {
    const int64_t xr = static_cast<int64_t>(set->data_bytes) / 4 / 4096 * 4096;
    if (xr >= (8 << 20)) {
      set->data_bytes -= static_cast<size_t>(2 * xr);
      if (ps.id == 0) {
        set->xchg_bytes = xr;
        set->xchg_off[0] = static_cast<int64_t>(set->data_bytes);
        set->xchg_off[1] = static_cast<int64_t>(set->data_bytes) + xr;
      }
    }
  }
  const size_t flag_words = static_cast<size_t>(SYMM_FLAG_BANKS) * SYMM_MAX_RANKS *
                            SYMM_MAX_BLOCKS;  // uint32 words per set
  for (int i = 0; i < set->world; ++i) {
    set->peers[i] = static_cast<char*>(a.peers[ranks[i]]);
    set->flags_peers[i] = a.flags[ranks[i]] + flag_words * ps.id;
  }
  set->local = set->peers[set->rank];
  set->flags_local = set->flags_peers[set->rank];
  set->nvls = a.multicast && set->world == a.world;
  set->mc = set->nvls ? static_cast<char*>(a.mc) : nullptr;
  // Fresh flag words for this set, agreed before anyone signals.
  HVD_CUDA(cudaMemsetAsync(set->flags_local, 0, flag_words * sizeof(uint32_t), stream_));
  HVD_CUDA(cudaStreamSynchronize(stream_));
  ps.comm.Barrier();
  SymmSet* raw = set.get();
  sets_[ps.id] = std::move(set);
  return raw;
}

kern::SymmCtx GpuOps::MakeCtx(SymmSet& set, uint32_t epochs, int64_t staging_off,
                              bool skip_end_barrier) {
  kern::SymmCtx c;
  std::memset(&c, 0, sizeof(c));
  c.rank = set.rank;
  c.world = set.world;
  c.local = set.local + staging_off;
  for (int i = 0; i < set.world; ++i) {
    c.peers[i] = set.peers[i] + staging_off;
    c.flags_peers[i] = set.flags_peers[i];
  }
  c.mc = set.mc ? set.mc + staging_off : nullptr;
  c.skip_end_barrier = skip_end_barrier ? 1 : 0;
  c.flags_local = set.flags_local;
  c.epoch = set.epoch;
  c.timeout_ns = timeout_ns_;
  c.status = status_dev_;
  c.trace = trace_dev_;
  set.epoch += epochs;
  return c;
}

Status GpuOps::CheckKernelStatus() {
  if (status_host_ != nullptr && status_host_->code == 2) {
    return Status::PreconditionError(
        "Rank " + std::to_string(status_host_->peer) +
        " did not pass the same symmetric-memory tensors to this collective. Tensors "
        "from hvd.symmetric_empty() must be used by all ranks alike (same allocation, "
        "same slices).");
  }
  if (status_host_ != nullptr && status_host_->code != 0) {
    return Status::UnknownError(
        "A collective kernel timed out waiting for rank " +
        std::to_string(status_host_->peer) + " (phase " +
        std::to_string(status_host_->phase) +
        "). The peer process probably died or stalled.");
  }
  return Status::OK();
}

int GpuOps::PickCtas(int64_t bytes) const {
  if (forced_ctas_ > 0) return std::min(forced_ctas_, SYMM_MAX_BLOCKS);
  // With several communication streams, kernels of different lanes may run
  // at the same time and each waits for its peers: all of them must be able
  // to be resident together (2 CTAs of 512 threads per SM on 148 SMs), or two
  // GPUs could each fill up with the kernel the other one is not running.
  const int cap = 296 / lanes_;
  auto capped = [cap](int n) { return std::min(n, cap); };
  // Few CTAs for latency-bound sizes, more as the message grows: a CTA keeps
  // about 32 KB of peer loads in flight, and NVLink needs a few MB in flight
  // to run at full rate.
  if (bytes <= 64 * 1024) return capped(4);
  if (bytes <= 512 << 10) return capped(16);
  if (bytes <= 2 << 20) return capped(32);
  if (bytes <= 8 << 20) return capped(64);
  if (bytes <= 32 << 20) return capped(96);
  if (bytes <= 128 << 20) return capped(148);
  return capped(296);  // two CTAs per SM: where the local copy phases peak
}

kern::Algo GpuOps::PickAlgo(const SymmSet& set, DataType wire,
                            int64_t bytes) const {
  if (set.world == 1) return kern::Algo::LOCAL;
  const bool nvls_type = wire == DataType::FLOAT32 || wire == DataType::FLOAT16 ||
                         wire == DataType::BFLOAT16;
  if (forced_algo_ == "oneshot") return kern::Algo::ONESHOT;
  if (forced_algo_ == "twoshot") return kern::Algo::TWOSHOT;
  if (forced_algo_ == "nvls" && set.nvls && nvls_type) return kern::Algo::NVLS;
  // One-shot costs one barrier less than two-shot but every rank reads all
  // of every peer's data: (N-1)S instead of 2S(N-1)/N over NVLink. With two
  // ranks that is the same traffic, so one-shot always wins there.
  int64_t oneshot_max = oneshot_max_;
  if (oneshot_max < 0)
    oneshot_max = set.world == 2 ? INT64_MAX : set.world <= 4 ? (2 << 20) : (512 << 10);
  if (bytes <= oneshot_max) return kern::Algo::ONESHOT;
  // Per-GPU NVLink traffic: NVLS moves S(N+1)/N each way, two-shot over peer
  // loads/stores 2S(N-1)/N, so the switch reduction wins from 4 ranks on.
  if (set.nvls && nvls_type && bytes >= nvls_min_ && set.world >= 4)
    return kern::Algo::NVLS;
  return kern::Algo::TWOSHOT;
}

void GpuOps::WaitForInputs(const std::vector<TensorTableEntry>& entries) {
  const ReadyEvent* last = nullptr;
  for (auto& e : entries) {
    if (e.ready && e.ready.get() != last) {
      e.ready->StreamWait(stream_);
      last = e.ready.get();
    }
  }
}

namespace {
double HostNowUs() {
  return std::chrono::duration<double, std::micro>(
             std::chrono::steady_clock::now().time_since_epoch()).count();
}
}  // namespace

cudaEvent_t GpuOps::TimedEvent() {
  {
    std::lock_guard<std::mutex> l(timed_mu_);
    if (!timed_events_.empty()) {
      cudaEvent_t e = timed_events_.back();
      timed_events_.pop_back();
      return e;
    }
  }
  cudaEvent_t e = nullptr;
  HVD_CUDA(cudaEventCreate(&e));
  return e;
}

void GpuOps::Calibrate() {
  // A completed event whose host time is known: later events are placed on
  // the host clock by their elapsed time since this one. Renewed every few
  // seconds so that the two clocks cannot drift apart noticeably.
  if (calib_event_ == nullptr) HVD_CUDA(cudaEventCreate(&calib_event_));
  HVD_CUDA(cudaEventRecord(calib_event_, stream_));
  HVD_CUDA(cudaEventSynchronize(calib_event_));
  calib_host_us_ = NowMicros();
}

int64_t GpuOps::EventHostMicros(cudaEvent_t ev) {
  float ms = 0.f;
  if (calib_event_ == nullptr || cudaEventElapsedTime(&ms, calib_event_, ev) != cudaSuccess) {
    cudaGetLastError();
    return NowMicros();
  }
  return calib_host_us_ + static_cast<int64_t>(ms * 1000.0);
}

void GpuOps::PushMark(std::vector<std::string> tensors, const char* activity) {
  if (marks_.empty() && (calib_event_ == nullptr || NowMicros() - calib_host_us_ > 5000000))
    Calibrate();
  ActivityMark m;
  m.tensors = std::move(tensors);
  m.activity = activity != nullptr ? activity : "";
  m.event = TimedEvent();
  HVD_CUDA(cudaEventRecord(m.event, stream_));
  marks_.push_back(std::move(m));
}

void GpuOps::ActStart(const std::vector<TensorTableEntry>& entries, const char* activity) {
  if (!state_.timeline.Initialized()) return;
  std::vector<std::string> names;
  for (auto& e : entries) names.push_back(e.name);
  PushMark(std::move(names), activity);
}

void GpuOps::ActEnd(const std::vector<TensorTableEntry>& entries) {
  if (!state_.timeline.Initialized()) return;
  std::vector<std::string> names;
  for (auto& e : entries) names.push_back(e.name);
  PushMark(std::move(names), nullptr);
}

void GpuOps::ActStart(const std::string& tensor, const char* activity) {
  if (!state_.timeline.Initialized()) return;
  PushMark({tensor}, activity);
}

void GpuOps::ActEnd(const std::string& tensor) {
  if (!state_.timeline.Initialized()) return;
  PushMark({tensor}, nullptr);
}

void GpuOps::CloseTiming() {
  PendingTiming* pt = open_timing_;
  if (pt == nullptr || pt->t1 == nullptr) return;
  open_timing_ = nullptr;
  host_trace::Mark("rest");
  cudaEventRecord(pt->t1, stream_);
  host_trace::Mark("end event");
  pt->host_us = static_cast<float>(HostNowUs() - pt->host_t0);
  std::lock_guard<std::mutex> l(timing_mu_);
  pending_timings_.push_back(*pt);
  pt->t1 = nullptr;
}

Status GpuOps::Complete(std::vector<TensorTableEntry>& entries) {
  CloseTiming();
  std::shared_ptr<void> done = events_->Get();
  HVD_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(done.get()), stream_));
  Timeline& tl = state_.timeline;
  if (async_completion_ && !tl.Initialized()) {
    Status st = CheckKernelStatus();
    for (auto& e : entries) e.Finish(st, done);
    return Status::InProgress();
  }
  // Host-synchronised completion: a finalizer thread waits for the event,
  // so errors and timeline end times belong to this very op.
  auto shared = std::make_shared<std::vector<TensorTableEntry>>(std::move(entries));
  entries.clear();
  auto marks = std::make_shared<std::vector<ActivityMark>>(std::move(marks_));
  marks_.clear();
  cudaEvent_t finished = nullptr;
  if (tl.Initialized()) {
    finished = TimedEvent();
    HVD_CUDA(cudaEventRecord(finished, stream_));
  }
  // Elastic jobs with NCCL communicators: poll instead of blocking, and ask
  // NCCL for asynchronous errors meanwhile; a peer that died then ends this
  // wait with an error (the communicators are aborted) instead of hanging it.
  NcclOps* watch = state_.elastic_enabled && nccl_ && nccl_->HasCommunicators() ? nccl_.get()
                                                                               : nullptr;
  finalizer_.Submit([this, shared, done, marks, finished, watch] {
    cudaEvent_t done_event = static_cast<cudaEvent_t>(done.get());
    cudaError_t err = cudaSuccess;
    Status async_status = Status::OK();
    if (watch != nullptr) {
      async_status = WaitPolling(
          [&] {
            cudaError_t q = cudaEventQuery(done_event);
            if (q == cudaSuccess) return 1;
            if (q == cudaErrorNotReady) return 0;
            err = q;
            return -1;
          },
          [&] { return watch->CheckAsyncErrors(); }, std::chrono::microseconds(200),
          std::chrono::milliseconds(5000));
    } else {
      err = cudaEventSynchronize(done_event);
    }
    Status st = err != cudaSuccess ? Status::UnknownError(std::string("CUDA error: ") +
                                                          cudaGetErrorString(err))
                : !async_status.ok() ? async_status
                                     : CheckKernelStatus();
    // Replay the phases with the times the device went through them (none
    // after an error: the events may never have completed).
    const bool timed = err == cudaSuccess && async_status.ok();
    Timeline& timeline = state_.timeline;
    for (auto& m : *marks) {
      const int64_t at = timed ? EventHostMicros(m.event) : -1;
      for (auto& name : m.tensors) {
        if (m.activity.empty())
          timeline.ActivityEndAt(name, at);
        else
          timeline.ActivityStartAt(name, m.activity, at);
      }
    }
    const int64_t end_at =
        finished != nullptr && timed ? EventHostMicros(finished) : -1;
    {
      std::lock_guard<std::mutex> l(timed_mu_);
      for (auto& m : *marks) timed_events_.push_back(m.event);
      if (finished != nullptr) timed_events_.push_back(finished);
    }
    for (auto& e : *shared) {
      timeline.EndAt(e.name, end_at);
      e.Finish(st, done);
    }
  });
  return Status::InProgress();
}

Status GpuOps::Execute(std::vector<TensorTableEntry>& entries,
                       const Response& response, ProcessSet& ps) {
  if (entries.empty()) return Status::OK();
  int device = -1;
  for (auto& e : entries)
    if (e.device != CPU_DEVICE_ID && (e.input || e.output)) device = e.device;
  if (device < 0) device = device_ >= 0 ? device_ : state_.config.local_rank;
  EnsureDevice(device);
  HVD_CUDA(cudaSetDevice(device_));
  Status pending = CheckKernelStatus();
  if (!pending.ok()) return pending;
  EnsureArena(ps);
  SymmSet* set = GetSymmSet(ps);

  const bool sum_like = response.reduce_op == ReduceOp::SUM ||
                        response.reduce_op == ReduceOp::AVERAGE ||
                        response.reduce_op == ReduceOp::ADASUM;
  bool use_symm = set != nullptr;
  if (use_symm) {
    switch (response.type) {
    case Response::ALLREDUCE:
    case Response::REDUCESCATTER:
      use_symm = sum_like && response.dtype != DataType::BOOL &&
                 response.dtype != DataType::INT16 &&
                 response.dtype != DataType::UINT16;
      break;
    case Response::ADASUM:
      use_symm = response.dtype == DataType::FLOAT32 ||
                 response.dtype == DataType::FLOAT16 ||
                 response.dtype == DataType::BFLOAT16;
      break;
    default:
      break;
    }
  }
  g_path_counts[use_symm ? 0 : 1].fetch_add(1, std::memory_order_relaxed);
  if (!use_symm && set != nullptr) {
    // The arena is there but this response cannot use it: say so once per kind.
    static std::atomic<unsigned> told{0};
    const unsigned bit = 1u << (static_cast<unsigned>(response.type) & 31u);
    if ((told.fetch_or(bit) & bit) == 0)
      HVD_LOG(INFO) << Response::TypeName(response.type) << " with reduce op "
                    << static_cast<int>(response.reduce_op) << " and dtype "
                    << DataTypeName(response.dtype)
                    << " runs on the NCCL path (the symmetric-memory kernels cover sum-like "
                       "reductions of every type but bool and 16-bit integers).";
  }
  PendingTiming pt = {nullptr, nullptr, static_cast<int>(response.type), 0,
                      static_cast<int>(entries.size()), 0.0, 0.f};
  if (timing_) {
    for (auto& e : entries) pt.bytes += e.size_bytes();
    WaitForInputs(entries);  // producer wait must not count as op time
    std::lock_guard<std::mutex> l(timing_mu_);
    for (cudaEvent_t* ev : {&pt.t0, &pt.t1}) {
      if (!timing_events_.empty()) {
        *ev = timing_events_.back();
        timing_events_.pop_back();
      } else {
        HVD_CUDA(cudaEventCreate(ev));
      }
    }
    HVD_CUDA(cudaEventRecord(pt.t0, stream_));
    pt.host_t0 = HostNowUs();
    open_timing_ = &pt;
    host_trace::Begin(static_cast<int>(response.type) + (use_symm ? 0 : 100));
  }
  // Normally Complete() closes the record right after the last launch; this
  // covers the paths that return without reaching it.
  struct TimingCloser {
    GpuOps* self;
    ~TimingCloser() {
      self->CloseTiming();
      self->open_timing_ = nullptr;
    }
  } closer{this};
  if (use_symm) {
    switch (response.type) {
    case Response::ALLREDUCE: return SymmAllreduce(entries, response, *set, false);
    case Response::ADASUM: return SymmAllreduce(entries, response, *set, true);
    case Response::BROADCAST: return SymmBroadcast(entries, *set);
    case Response::ALLGATHER: return SymmAllgather(entries, response, *set);
    case Response::ALLTOALL: return SymmAlltoall(entries, response, ps, *set);
    case Response::REDUCESCATTER: return SymmReducescatter(entries, *set);
    default: break;
    }
  }
  if (!nccl_) nccl_.reset(new NcclOps(*this));
  return nccl_->Execute(entries, response, ps);
}

void* GpuOps::SymmHeapAlloc(size_t bytes, int64_t* offset) {
  if (!arena_.valid() || heap_bytes_ == 0) return nullptr;
  const int64_t need = RoundUp(static_cast<int64_t>(bytes), 256);
  int64_t at = heap_used_.fetch_add(need);
  if (at + need > heap_bytes_) {
    heap_used_.fetch_sub(need);
    return nullptr;
  }
  if (offset) *offset = heap_off_ + at;
  return heap_base_ + at;
}

bool GpuOps::InSymmHeap(const void* p, int64_t bytes, int64_t* offset) const {
  if (heap_base_ == nullptr) return false;
  const char* c = static_cast<const char*>(p);
  if (c < heap_base_ || c + bytes > heap_base_ + heap_used_.load()) return false;
  if (offset) *offset = heap_off_ + (c - heap_base_);
  return true;
}

std::vector<GpuOps::OpTiming> GpuOps::DrainTimings() {
  std::vector<PendingTiming> pending;
  {
    std::lock_guard<std::mutex> l(timing_mu_);
    pending.swap(pending_timings_);
  }
  std::vector<OpTiming> out;
  for (auto& p : pending) {
    OpTiming t = {p.type, p.bytes, p.tensors, 0.f, p.host_us};
    float ms = 0.f;
    if (cudaEventSynchronize(p.t1) == cudaSuccess &&
        cudaEventElapsedTime(&ms, p.t0, p.t1) == cudaSuccess)
      t.device_us = ms * 1000.f;
    out.push_back(t);
    std::lock_guard<std::mutex> l(timing_mu_);
    timing_events_.push_back(p.t0);
    timing_events_.push_back(p.t1);
  }
  return out;
}

void GpuOps::Shutdown() {
  if (shut_down_) return;
  shut_down_ = true;
  if (slot_ == 0 && lane_ == 0) host_trace::Report(state_.config.rank);
  GpuOps* self = this;
  g_current.compare_exchange_strong(self, nullptr);
  {
    std::lock_guard<std::mutex> l(g_registry_mu_ref());
    auto& reg = g_registry_ref();
    reg.erase(std::remove(reg.begin(), reg.end(), this), reg.end());
  }
  if (device_ >= 0) {
    cudaSetDevice(device_);
    if (stream_) cudaStreamSynchronize(stream_);
  }
  finalizer_.Shutdown();
  if (nccl_) nccl_->Shutdown();
  nccl_.reset();
  sets_.clear();
  // Every rank reaches this point through the coordinated shutdown, after
  // its last kernel finished. Meet once more on the control plane so that
  // no rank unmaps memory a slower peer's last kernel may still read; if a
  // peer is gone already there is nobody left to protect.
  if (arena_.valid() && state_.config.size > 1) {
    try {
      state_.process_sets.Get(0).comm.Barrier();
    } catch (const std::exception&) {
    }
  }
  arena_.Destroy();
  heap_base_ = nullptr;
  heap_bytes_ = 0;
  ring_.Destroy();
  if (status_host_) cudaFreeHost(status_host_);
  status_host_ = nullptr;
  if (tile_counter_) cudaFree(tile_counter_);
  tile_counter_ = nullptr;
  if (xchg_done_counter_) cudaFree(xchg_done_counter_);
  xchg_done_counter_ = nullptr;
  if (trace_host_) cudaFreeHost(trace_host_);
  trace_host_ = nullptr;
  trace_dev_ = nullptr;
  if (stream_) cudaStreamDestroy(stream_);
  stream_ = nullptr;
  SetGpuBackendDescription("none");
}

}  // namespace hvd
