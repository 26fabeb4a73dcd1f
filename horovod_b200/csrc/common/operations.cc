#include "operations.h"

#include <chrono>
#include <stdexcept>

#include "../ops/cpu_ops.h"
#include "env.h"
#include "logging.h"
#include "nvtx_op_range.h"

namespace hvd {

namespace {

GlobalState g_state;
GpuOpsFactory g_gpu_factory;

const char* const NOT_INITIALIZED_MESSAGE =
    "Horovod has not been initialized; use hvd.init().";

Status CheckRunning() {
  if (!g_state.initialization_done.load() || g_state.loop_exited.load()) {
    std::lock_guard<std::mutex> l(g_state.error_mu);
    if (!g_state.fatal_error.empty())
      return Status::UnknownError(g_state.fatal_error);
    if (g_state.shut_down.load())
      return Status::Aborted(SHUT_DOWN_ERROR_MESSAGE);
    return Status::PreconditionError(NOT_INITIALIZED_MESSAGE);
  }
  if (g_state.shut_down.load()) return Status::Aborted(SHUT_DOWN_ERROR_MESSAGE);
  return Status::OK();
}

void PerformOperation(GlobalState& s, ProcessSet& ps, const Response& response) {
  std::vector<TensorTableEntry> entries;
  ps.tensor_queue.GetTensorEntriesFromResponse(response, entries, ps.join.joined);

  if (response.type == Response::JOIN) {
    ps.join.joined = false;
    ps.join.last_joined_rank = -1;
    for (auto& e : entries) {
      if (e.output != nullptr)
        *static_cast<int32_t*>(e.output) = response.last_joined_rank;
      e.Finish(Status::OK());
    }
    return;
  }

  if (s.timeline.Initialized())
    for (auto& e : entries)
      s.timeline.Start(e.name, response.type, e.size_bytes());
  ps.group_table.DeregisterGroups(response.names);

  Status st;
  if (response.type == Response::ERROR) {
    st = Status::PreconditionError(response.error_message);
  } else {
    try {
      bool on_cpu = entries.empty() || entries[0].device == CPU_DEVICE_ID;
      // Joined stand-ins inherit the device of the ranks that have data.
      OpExecutor* ex = on_cpu ? s.cpu_ops.get() : s.gpu_ops.get();
      if (ex == nullptr)
        st = Status::PreconditionError(
            "A collective was requested on a CUDA tensor but this process has "
            "no usable GPU executor.");
      else
        st = ex->Execute(entries, response, ps);
    } catch (const TransportError&) {
      throw;  // ranks may now disagree about what ran: take the loop down
    } catch (const std::exception& e) {
      st = Status::UnknownError(e.what());
    }
  }
  if (!st.in_progress()) {
    if (s.timeline.Initialized())
      for (auto& e : entries) s.timeline.End(e.name);
    for (auto& e : entries) e.Finish(st);
  }
}

// Applies add/remove requests once every rank has the same one pending.
void CoordinateProcessSetChanges(GlobalState& s) {
  std::shared_ptr<GlobalState::PendingSetChange> head;
  {
    std::lock_guard<std::mutex> l(s.ctl_mu);
    if (!s.pending_set_changes.empty()) head = s.pending_set_changes.front();
  }
  int64_t mine[2] = {0, 0};
  if (head) {
    if (head->add) {
      mine[0] = 1;
      uint64_t h = 1469598103934665603ull;  // FNV-1a over the rank list
      for (int r : head->ranks) {
        h ^= static_cast<uint64_t>(r) + 1;
        h *= 1099511628211ull;
      }
      mine[1] = static_cast<int64_t>(h >> 1);
    } else {
      mine[0] = 2;
      mine[1] = head->id;
    }
  }
  Comm& world = s.process_sets.Get(0).comm;
  std::vector<int64_t> all(2 * world.size());
  world.Allgather(mine, sizeof(mine), all.data());
  if (!head) return;
  for (int r = 0; r < world.size(); ++r)
    if (all[2 * r] != mine[0] || all[2 * r + 1] != mine[1]) return;  // wait
  try {
    if (head->add) {
      head->id = s.process_sets.RegisterProcessSet(head->ranks);
    } else {
      s.process_sets.DeregisterProcessSet(head->id);
    }
  } catch (const std::exception& e) {
    head->error = e.what();
  }
  {
    std::lock_guard<std::mutex> l(s.ctl_mu);
    s.pending_set_changes.erase(s.pending_set_changes.begin());
    head->done = true;
  }
  s.ctl_cv.notify_all();
}

bool RunLoopOnce(GlobalState& s,
                 std::chrono::steady_clock::time_point& last_cycle) {
  auto cycle = std::chrono::duration<double, std::milli>(
      s.parameter_manager.CycleTimeMs());
  auto next = last_cycle +
              std::chrono::duration_cast<std::chrono::steady_clock::duration>(cycle);
  auto now = std::chrono::steady_clock::now();
  if (next > now) {
    if (s.flush_on_wait) {
      // Sleep out the cycle unless somebody blocks in synchronize(): then the
      // next negotiation starts at once (after a short pause, so that a long
      // wait does not turn into a busy loop of control-plane rounds). The
      // cycle time exists to batch tensors for fusion; a caller that is
      // already waiting has nothing more to add to the batch.
      const auto floor = last_cycle + std::chrono::microseconds(50);
      std::unique_lock<std::mutex> l(s.wake_mu);
      s.wake_cv.wait_until(l, next, [&s] { return s.sync_waiters.load() > 0; });
      l.unlock();
      now = std::chrono::steady_clock::now();
      if (now < floor) std::this_thread::sleep_until(floor);
    } else {
      std::this_thread::sleep_until(next);
    }
  }
  last_cycle = std::chrono::steady_clock::now();

  {
    std::lock_guard<std::mutex> l(s.ctl_mu);
    if (s.pending_timeline_stop) {
      s.timeline.Shutdown();
      s.pending_timeline_stop = false;
    }
    if (s.pending_timeline_start) {
      if (s.config.rank == 0)
        s.timeline.Initialize(s.pending_timeline_file,
                              s.pending_timeline_mark_cycles);
      s.pending_timeline_start = false;
    }
  }
  s.timeline.MarkCycleStart();

  if (s.dynamic_process_sets) CoordinateProcessSetChanges(s);

  bool keep_running = true;
  for (int32_t id : s.process_sets.Ids()) {
    ProcessSet& ps = s.process_sets.Get(id);
    if (!ps.IsCurrentProcessIncluded()) continue;
    ResponseList rl =
        ps.controller.ComputeResponseList(s.shut_down.load(), ps.join);

    std::vector<std::string> names;
    int64_t bytes = 0;
    bool tuning = id == 0 && s.parameter_manager.IsAutoTuning();
    if (tuning) bytes = ps.tensor_queue.GetTensorDataForAutotuner(rl, names);

    for (auto& response : rl.responses) PerformOperation(s, ps, response);

    if (tuning && s.parameter_manager.Update(names, bytes))
      ps.controller.SynchronizeParameters();
    if (rl.shutdown) keep_running = false;
  }
  return keep_running;
}

void DiscoverLayout(GlobalState& s) {
  Comm& world = s.process_sets.Get(0).comm;
  std::vector<int32_t> sizes(world.size());
  int32_t mine = s.config.local_size;
  world.Allgather(&mine, sizeof(mine), sizes.data());
  s.local_sizes.assign(sizes.begin(), sizes.end());
  s.is_homogeneous = true;
  for (auto v : sizes)
    if (v != sizes[0]) s.is_homogeneous = false;
  // Who sits where: (cross_rank, local_rank) of every rank.
  std::vector<int32_t> place(static_cast<size_t>(world.size()) * 2);
  int32_t me[2] = {s.config.cross_rank, s.config.local_rank};
  world.Allgather(me, sizeof(me), place.data());
  std::vector<int> same_host, same_slot;
  bool host_major = s.is_homogeneous;
  for (int r = 0; r < world.size(); ++r) {
    if (place[2 * r] == s.config.cross_rank) same_host.push_back(r);
    if (place[2 * r + 1] == s.config.local_rank) same_slot.push_back(r);
    if (r != place[2 * r] * s.config.local_size + place[2 * r + 1]) host_major = false;
  }
  s.local_comm = world.Subset(same_host);
  s.cross_comm = world.Subset(same_slot);
  s.hierarchy_usable = host_major && s.config.local_size > 1 && s.config.cross_size > 1 &&
                       static_cast<int>(same_host.size()) == s.config.local_size &&
                       static_cast<int>(same_slot.size()) == s.config.cross_size;
}

void BackgroundThreadLoop(GlobalState& s) {
  SetLogRank(s.config.rank);
  try {
    SetThreadAffinity(AffinityCore(EnvString(HVD_ENV_THREAD_AFFINITY), s.config.local_rank));
    double timeout = EnvDouble(HVD_ENV_TIMEOUT_SECONDS, 30.0);
    s.mesh.set_timeout(timeout);
    if (s.config.size > 1) {
      s.mesh.Connect(s.config.rank, s.config.size, s.config.peer_addrs,
                     s.config.token, std::max(timeout, 60.0));
    } else {
      s.mesh.Connect(0, 1, {std::string("localhost:0")}, s.config.token, 1.0);
    }

    // Knobs. A value given explicitly is pinned; the autotuner leaves it.
    s.parameter_manager = ParameterManager();
    ParameterManager& pm = s.parameter_manager;
    pm.SetTensorFusionThresholdBytes(
        EnvInt(HVD_ENV_FUSION_THRESHOLD, 128ll * 1024 * 1024),
        EnvIsSet(HVD_ENV_FUSION_THRESHOLD));
    s.flush_on_wait = EnvBool("HOROVOD_FLUSH_ON_WAIT", true);
    pm.SetCycleTimeMs(EnvDouble(HVD_ENV_CYCLE_TIME, 1.0),
                      EnvIsSet(HVD_ENV_CYCLE_TIME));
    uint32_t cache_capacity =
        static_cast<uint32_t>(EnvInt(HVD_ENV_CACHE_CAPACITY, 1024));
    pm.SetCacheEnabled(cache_capacity > 0, EnvIsSet(HVD_ENV_CACHE_CAPACITY));
    pm.SetHierarchicalAllreduce(EnvBool(HVD_ENV_HIERARCHICAL_ALLREDUCE, false),
                                true);
    pm.SetHierarchicalAllgather(EnvBool(HVD_ENV_HIERARCHICAL_ALLGATHER, false),
                                true);
    pm.SetWarmupSamples(static_cast<int>(EnvInt(HVD_ENV_AUTOTUNE_WARMUP_SAMPLES, 3)));
    pm.SetStepsPerSample(static_cast<int>(EnvInt(HVD_ENV_AUTOTUNE_STEPS_PER_SAMPLE, 10)));
    pm.SetBayesOptMaxSamples(static_cast<int>(EnvInt(HVD_ENV_AUTOTUNE_BAYES_OPT_MAX_SAMPLES, 20)));
    pm.SetGaussianProcessNoise(EnvDouble(HVD_ENV_AUTOTUNE_GAUSSIAN_PROCESS_NOISE, 0.8));
    pm.Initialize(s.config.rank, 0, EnvString(HVD_ENV_AUTOTUNE_LOG));

    ControllerOptions opts;
    opts.fusion_threshold_bytes = pm.TensorFusionThresholdBytes();
    opts.disable_group_fusion = EnvBool(HVD_ENV_DISABLE_GROUP_FUSION, false);
    opts.cache_capacity = cache_capacity;
    opts.local_size = s.config.local_size;
    bool stall_check = !EnvBool(HVD_ENV_STALL_CHECK_DISABLE, false);
    int warn_s = static_cast<int>(EnvInt(HVD_ENV_STALL_CHECK_TIME, 60));
    int shutdown_s = static_cast<int>(EnvInt(HVD_ENV_STALL_SHUTDOWN_TIME, 0));
    if (shutdown_s > 0 && shutdown_s < warn_s) {
      HVD_LOG(WARNING) << HVD_ENV_STALL_SHUTDOWN_TIME
                       << " is below the warning time; raising it to " << warn_s;
      shutdown_s = warn_s;
    }
    s.process_sets.Initialize(&s.mesh, &s.timeline, &s.parameter_manager, opts,
                              stall_check, warn_s, shutdown_s);
    for (auto& ranks : s.config.process_sets)
      s.process_sets.RegisterProcessSet(ranks);
    DiscoverLayout(s);

    s.elastic_enabled = EnvBool(HVD_ENV_ELASTIC, false);
    NvtxSetEnabled(!EnvBool(HVD_ENV_DISABLE_NVTX, false));
    s.dynamic_process_sets = EnvBool("HOROVOD_DYNAMIC_PROCESS_SETS", false);

    std::string tl = EnvString(HVD_ENV_TIMELINE);
    s.timeline_mark_cycles = EnvBool(HVD_ENV_TIMELINE_MARK_CYCLES, false);
    if (!tl.empty() && tl != "DYNAMIC" && s.config.rank == 0)
      s.timeline.Initialize(tl, s.timeline_mark_cycles);

    s.cpu_ops = MakeCpuOps(s);
    s.gpu_ops.reset();
    if (g_gpu_factory) s.gpu_ops = g_gpu_factory(s);

    if (EnvBool(HVD_ENV_AUTOTUNE, false)) {
      pm.SetAutoTuning(true);
      s.process_sets.Get(0).controller.SynchronizeParameters();
    }
    s.process_sets.Get(0).comm.Barrier();
  } catch (const std::exception& e) {
    s.init_error = e.what();
    s.mesh.Close();
    s.loop_exited = true;
    s.init_failed = true;
    return;
  }
  s.loop_exited = false;
  s.initialization_done = true;
  HVD_LOG(DEBUG) << "background loop running (size " << s.config.size << ")";

  auto last_cycle = std::chrono::steady_clock::now();
  std::string fatal;
  try {
    while (RunLoopOnce(s, last_cycle)) {
    }
  } catch (const std::exception& e) {
    fatal = e.what();
    HVD_LOG(ERROR) << "Horovod background loop failed: " << fatal;
  }

  // Ordered teardown. Whatever is still pending can never complete.
  {
    std::lock_guard<std::mutex> l(s.error_mu);
    s.fatal_error = fatal;
  }
  s.shut_down = true;
  Status final_status = fatal.empty()
                            ? Status::Aborted(SHUT_DOWN_ERROR_MESSAGE)
                            : Status::UnknownError(fatal);
  if (s.gpu_ops) s.gpu_ops->Shutdown();
  for (int32_t id : s.process_sets.Ids())
    s.process_sets.Get(id).tensor_queue.FinalizeTensorQueue(final_status);
  {
    std::lock_guard<std::mutex> l(s.ctl_mu);
    for (auto& c : s.pending_set_changes) {
      c->error = "Horovod has been shut down.";
      c->done = true;
    }
    s.pending_set_changes.clear();
  }
  s.ctl_cv.notify_all();
  s.timeline.Shutdown();
  s.gpu_ops.reset();
  s.cpu_ops.reset();
  s.mesh.Close();
  s.loop_exited = true;
}

}  // namespace

GlobalState& hvd_state() { return g_state; }

void hvd_set_gpu_ops_factory(GpuOpsFactory f) { g_gpu_factory = std::move(f); }

std::string hvd_listen(const std::string& advertise_host) {
  if (g_state.initialization_done.load() && !g_state.loop_exited.load())
    throw std::runtime_error("hvd: already initialised");
  return g_state.mesh.Listen(advertise_host);
}

void hvd_init(const InitConfig& cfg) {
  GlobalState& s = g_state;
  if (s.initialization_done.load() && !s.loop_exited.load()) return;
  if (s.background_thread.joinable()) s.background_thread.join();
  ResetLogLevelFromEnv();
  s.config = cfg;
  s.initialization_done = false;
  s.init_failed = false;
  s.init_error.clear();
  s.shut_down = false;
  {
    std::lock_guard<std::mutex> l(s.error_mu);
    s.fatal_error.clear();
  }
  s.background_thread = std::thread([&s] { BackgroundThreadLoop(s); });
  while (!s.initialization_done.load() && !s.init_failed.load())
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  if (s.init_failed.load()) {
    s.background_thread.join();
    throw std::runtime_error("Horovod initialization failed: " + s.init_error);
  }
}

void hvd_shutdown() {
  GlobalState& s = g_state;
  s.shut_down = true;
  if (s.background_thread.joinable()) s.background_thread.join();
  // Re-arm so that init can run again (elastic reset).
  s.initialization_done = false;
  s.process_sets.Clear();
}

void hvd_waiter_enter() {
  GlobalState& s = g_state;
  {
    std::lock_guard<std::mutex> l(s.wake_mu);
    s.sync_waiters.fetch_add(1);
  }
  s.wake_cv.notify_all();
}

void hvd_waiter_exit() { g_state.sync_waiters.fetch_sub(1); }

bool hvd_is_initialized() {
  return g_state.initialization_done.load() && !g_state.loop_exited.load();
}

// True from init() until shutdown(), also after the background loop has ended
// because a peer shut the job down: rank()/size() stay answerable then, as in
// the reference (horovod_rank() only checks initialization_done,
// horovod/common/operations.cc:1043-1049).
bool hvd_has_topology() { return g_state.initialization_done.load(); }

namespace {
void RequireInit() {
  if (!g_state.initialization_done.load())
    throw std::runtime_error(NOT_INITIALIZED_MESSAGE);
}
}  // namespace

int hvd_rank() { RequireInit(); return g_state.config.rank; }
int hvd_size() { RequireInit(); return g_state.config.size; }
int hvd_local_rank() { RequireInit(); return g_state.config.local_rank; }
int hvd_local_size() { RequireInit(); return g_state.config.local_size; }
int hvd_cross_rank() { RequireInit(); return g_state.config.cross_rank; }
int hvd_cross_size() { RequireInit(); return g_state.config.cross_size; }
bool hvd_is_homogeneous() { RequireInit(); return g_state.is_homogeneous; }

void hvd_start_timeline(const std::string& file, bool mark_cycles) {
  RequireInit();
  std::lock_guard<std::mutex> l(g_state.ctl_mu);
  g_state.pending_timeline_file = file;
  g_state.pending_timeline_mark_cycles = mark_cycles;
  g_state.pending_timeline_start = true;
}

void hvd_stop_timeline() {
  RequireInit();
  std::lock_guard<std::mutex> l(g_state.ctl_mu);
  g_state.pending_timeline_stop = true;
  g_state.pending_timeline_start = false;
}

int32_t hvd_add_process_set(const std::vector<int>& ranks) {
  RequireInit();
  GlobalState& s = g_state;
  if (!s.dynamic_process_sets)
    throw std::runtime_error(
        "Process sets can only be added after init when "
        "HOROVOD_DYNAMIC_PROCESS_SETS=1 is set; otherwise pass them to "
        "hvd.init(process_sets=...).");
  auto change = std::make_shared<GlobalState::PendingSetChange>();
  change->add = true;
  change->ranks = ranks;
  change->id = -1;
  std::unique_lock<std::mutex> l(s.ctl_mu);
  s.pending_set_changes.push_back(change);
  s.ctl_cv.wait(l, [&] { return change->done; });
  if (!change->error.empty()) throw std::runtime_error(change->error);
  return change->id;
}

void hvd_remove_process_set(int32_t id) {
  RequireInit();
  GlobalState& s = g_state;
  if (!s.dynamic_process_sets)
    throw std::runtime_error(
        "Process sets can only be removed when HOROVOD_DYNAMIC_PROCESS_SETS=1 "
        "is set.");
  auto change = std::make_shared<GlobalState::PendingSetChange>();
  change->add = false;
  change->id = id;
  std::unique_lock<std::mutex> l(s.ctl_mu);
  s.pending_set_changes.push_back(change);
  s.ctl_cv.wait(l, [&] { return change->done; });
  if (!change->error.empty()) throw std::runtime_error(change->error);
}

int hvd_process_set_rank(int32_t id) {
  RequireInit();
  return g_state.process_sets.Get(id).comm.rank();
}
int hvd_process_set_size(int32_t id) {
  RequireInit();
  return g_state.process_sets.Get(id).comm.size();
}
bool hvd_process_set_included(int32_t id) {
  RequireInit();
  return g_state.process_sets.Get(id).IsCurrentProcessIncluded();
}
std::vector<int> hvd_process_set_ranks(int32_t id) {
  RequireInit();
  return g_state.process_sets.Get(id).ranks();
}
std::vector<int32_t> hvd_process_set_ids() {
  RequireInit();
  return g_state.process_sets.Ids();
}

// ---------------------------------------------------------------------------
// Enqueue API

namespace {

Status FindSet(int32_t id, ProcessSet** out) {
  Status st = CheckRunning();
  if (!st.ok()) return st;
  if (!g_state.process_sets.Contains(id))
    return Status::InvalidArgument("Process set with id " + std::to_string(id) +
                                   " does not exist.");
  ProcessSet& ps = g_state.process_sets.Get(id);
  if (!ps.IsCurrentProcessIncluded())
    return Status::InvalidArgument(
        "This rank is not a member of process set " + std::to_string(id) + ".");
  *out = &ps;
  return Status::OK();
}

// Opens an NVTX range now and closes it when the entry completes.
void AttachNvtxRange(TensorTableEntry& e, NvtxOp op) {
  NvtxRangeId id = NvtxRangeStart(op, e.name, e.size_bytes());
  if (id == 0) return;
  StatusCallback inner = std::move(e.callback);
  e.callback = [inner, id](const Completion& c) {
    NvtxRangeEnd(id);
    if (inner) inner(c);
  };
}

Request MakeRequest(const TensorTableEntry& e, Request::Type type, int rank) {
  Request q;
  q.request_rank = rank;
  q.type = type;
  q.dtype = e.dtype;
  q.name = e.name;
  q.root_rank = e.root_rank;
  q.device = e.device;
  q.group_id = e.group_id;
  q.reduce_op = e.reduce_op;
  q.shape = e.shape.to_vector();
  q.prescale = e.prescale;
  q.postscale = e.postscale;
  q.wire_dtype = e.wire_dtype;
  return q;
}

}  // namespace

Status EnqueueTensorAllreduces(std::vector<TensorTableEntry>& entries,
                               ReduceOp op, double prescale, double postscale,
                               int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  if (entries.empty()) return Status::OK();

  Request::Type type = Request::ALLREDUCE;
  ReduceOp wire_op = op;
  if (op == ReduceOp::AVERAGE) {
    // Averaging is a sum whose post-scale carries the 1/size.
    wire_op = ReduceOp::SUM;
    postscale /= ps->comm.size();
  } else if (op == ReduceOp::ADASUM) {
    type = Request::ADASUM;
  }
  int32_t group_id = NULL_GROUP_ID;
  if (entries.size() > 1) {
    std::vector<std::string> names;
    for (auto& e : entries) names.push_back(e.name);
    group_id = ps->group_table.RegisterGroup(std::move(names));
  }
  std::vector<Request> requests;
  int64_t now = NowMicros();
  for (auto& e : entries) {
    const bool cast_ok = e.dtype == DataType::FLOAT32 && e.device != CPU_DEVICE_ID &&
                         (e.wire_dtype == DataType::FLOAT16 ||
                          e.wire_dtype == DataType::BFLOAT16) &&
                         type == Request::ALLREDUCE;
    if (!cast_ok) e.wire_dtype = e.dtype;
    e.reduce_op = wire_op;
    e.prescale = prescale;
    e.postscale = postscale;
    e.process_set_id = process_set_id;
    e.group_id = group_id;
    e.enqueue_us = now;
    AttachNvtxRange(e, entries.size() > 1 ? NvtxOp::GROUPED_ALLREDUCE : NvtxOp::ALLREDUCE);
    requests.push_back(MakeRequest(e, type, ps->comm.rank()));
  }
  st = ps->tensor_queue.AddToTensorQueueMulti(entries, requests);
  if (!st.ok() && group_id != NULL_GROUP_ID) {
    std::vector<std::string> names;
    for (auto& q : requests) names.push_back(q.name);
    ps->group_table.DeregisterGroups(names);
  }
  return st;
}

Status EnqueueTensorAllgather(TensorTableEntry entry, int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  entry.process_set_id = process_set_id;
  entry.enqueue_us = NowMicros();
  AttachNvtxRange(entry, NvtxOp::ALLGATHER);
  Request q = MakeRequest(entry, Request::ALLGATHER, ps->comm.rank());
  return ps->tensor_queue.AddToTensorQueue(std::move(entry), std::move(q));
}

Status EnqueueTensorBroadcast(TensorTableEntry entry, int root_rank,
                              int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  // The API takes a global rank; ops work with set-relative ranks.
  int set_root = -1;
  const auto& ranks = ps->ranks();
  for (size_t i = 0; i < ranks.size(); ++i)
    if (ranks[i] == root_rank) set_root = static_cast<int>(i);
  if (set_root < 0)
    return Status::InvalidArgument(
        "broadcast received invalid root rank " + std::to_string(root_rank) +
        " for process set " + std::to_string(process_set_id) + ".");
  entry.root_rank = set_root;
  entry.process_set_id = process_set_id;
  entry.enqueue_us = NowMicros();
  AttachNvtxRange(entry, NvtxOp::BROADCAST);
  Request q = MakeRequest(entry, Request::BROADCAST, ps->comm.rank());
  return ps->tensor_queue.AddToTensorQueue(std::move(entry), std::move(q));
}

Status EnqueueTensorAlltoall(TensorTableEntry entry, int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  int n = ps->comm.size();
  if (entry.shape.dims() == 0)
    return Status::InvalidArgument("alltoall needs a tensor of rank 1 or more.");
  int64_t rows = entry.shape.dim_size(0);
  // For an alltoall the root_rank field of the request says whether this rank
  // left the splits to the library (1: even split). When every rank did, the
  // response carries every rank's first dimension and nobody has to exchange
  // split tables before the data.
  entry.root_rank = entry.splits.empty() ? 1 : 0;
  if (entry.splits.empty()) {
    if (rows % n != 0)
      return Status::InvalidArgument(
          "splits not provided to alltoall and the first dimension of the "
          "tensor (" + std::to_string(rows) +
          ") is not a multiple of the number of ranks (" + std::to_string(n) + ").");
    entry.splits.assign(n, static_cast<int32_t>(rows / n));
  } else {
    if (static_cast<int>(entry.splits.size()) != n)
      return Status::InvalidArgument(
          "Number of entries in splits (" + std::to_string(entry.splits.size()) +
          ") must equal the number of ranks (" + std::to_string(n) + ").");
    int64_t sum = 0;
    for (auto v : entry.splits) {
      if (v < 0) return Status::InvalidArgument("Negative entry in alltoall splits.");
      sum += v;
    }
    if (sum > rows)
      return Status::InvalidArgument(
          "Sum of splits entries is greater than the first dimension of tensor.");
  }
  entry.process_set_id = process_set_id;
  entry.enqueue_us = NowMicros();
  AttachNvtxRange(entry, NvtxOp::ALLTOALL);
  Request q = MakeRequest(entry, Request::ALLTOALL, ps->comm.rank());
  return ps->tensor_queue.AddToTensorQueue(std::move(entry), std::move(q));
}

Status EnqueueTensorReducescatter(TensorTableEntry entry, ReduceOp op,
                                  double prescale, double postscale,
                                  int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  if (op == ReduceOp::ADASUM)
    return Status::InvalidArgument("reducescatter does not support Adasum.");
  if (op == ReduceOp::AVERAGE) {
    op = ReduceOp::SUM;
    postscale /= ps->comm.size();
  }
  entry.reduce_op = op;
  entry.prescale = prescale;
  entry.postscale = postscale;
  entry.process_set_id = process_set_id;
  entry.enqueue_us = NowMicros();
  AttachNvtxRange(entry, NvtxOp::REDUCESCATTER);
  Request q = MakeRequest(entry, Request::REDUCESCATTER, ps->comm.rank());
  return ps->tensor_queue.AddToTensorQueue(std::move(entry), std::move(q));
}

namespace {
// Enqueues several entries of one kind as a group: the controller keeps the
// members together, so they are negotiated in one cycle and fused into one
// response (horovod/common/operations.cc EnqueueTensorAllreduces registers
// its groups the same way).
Status EnqueueGroup(ProcessSet* ps, std::vector<TensorTableEntry>& entries,
                    Request::Type type, NvtxOp nvtx) {
  int32_t group_id = NULL_GROUP_ID;
  if (entries.size() > 1) {
    std::vector<std::string> names;
    for (auto& e : entries) names.push_back(e.name);
    group_id = ps->group_table.RegisterGroup(std::move(names));
  }
  std::vector<Request> requests;
  const int64_t now = NowMicros();
  for (auto& e : entries) {
    e.group_id = group_id;
    e.enqueue_us = now;
    AttachNvtxRange(e, nvtx);
    requests.push_back(MakeRequest(e, type, ps->comm.rank()));
  }
  Status st = ps->tensor_queue.AddToTensorQueueMulti(entries, requests);
  if (!st.ok() && group_id != NULL_GROUP_ID) {
    std::vector<std::string> names;
    for (auto& q : requests) names.push_back(q.name);
    ps->group_table.DeregisterGroups(names);
  }
  return st;
}
}  // namespace

Status EnqueueTensorAllgathers(std::vector<TensorTableEntry>& entries,
                               int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  if (entries.empty()) return Status::OK();
  for (auto& e : entries) e.process_set_id = process_set_id;
  return EnqueueGroup(ps, entries, Request::ALLGATHER, NvtxOp::ALLGATHER);
}

Status EnqueueTensorReducescatters(std::vector<TensorTableEntry>& entries, ReduceOp op,
                                   double prescale, double postscale,
                                   int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  if (entries.empty()) return Status::OK();
  if (op == ReduceOp::ADASUM)
    return Status::InvalidArgument("reducescatter does not support Adasum.");
  if (op == ReduceOp::AVERAGE) {
    op = ReduceOp::SUM;
    postscale /= ps->comm.size();
  }
  for (auto& e : entries) {
    e.reduce_op = op;
    e.prescale = prescale;
    e.postscale = postscale;
    e.process_set_id = process_set_id;
  }
  return EnqueueGroup(ps, entries, Request::REDUCESCATTER, NvtxOp::REDUCESCATTER);
}

Status EnqueueJoin(TensorTableEntry entry, int32_t process_set_id) {
  ProcessSet* ps = nullptr;
  Status st = FindSet(process_set_id, &ps);
  if (!st.ok()) return st;
  entry.name = JOIN_TENSOR_NAME;
  entry.process_set_id = process_set_id;
  entry.enqueue_us = NowMicros();
  Request q = MakeRequest(entry, Request::JOIN, ps->comm.rank());
  return ps->tensor_queue.AddToTensorQueue(std::move(entry), std::move(q));
}

}  // namespace hvd
