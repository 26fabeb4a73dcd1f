#include "timeline.h"

#include "logging.h"
#include "nvtx_op_range.h"

namespace hvd {

namespace {
std::string JsonEscape(const std::string& s) {
  std::string o;
  o.reserve(s.size() + 2);
  for (char c : s) {
    switch (c) {
    case '"': o += "\\\""; break;
    case '\\': o += "\\\\"; break;
    case '\n': o += "\\n"; break;
    case '\t': o += "\\t"; break;
    default:
      if (static_cast<unsigned char>(c) < 0x20) o += ' ';
      else o += c;
    }
  }
  return o;
}
}  // namespace

void Timeline::Initialize(const std::string& file, bool mark_cycles) {
  if (active_.load()) return;
  if (writer_.joinable()) writer_.join();
  file_ = std::fopen(file.c_str(), "w");
  if (file_ == nullptr) {
    HVD_LOG(ERROR) << "Cannot open timeline file " << file;
    return;
  }
  std::fputs("[\n", file_);
  first_event_ = true;
  tensor_pid_.clear();
  {
    std::lock_guard<std::mutex> l(state_mu_);
    states_.clear();
  }
  {
    std::lock_guard<std::mutex> l(q_mu_);
    queue_.clear();
    stop_ = false;
  }
  mark_cycles_ = mark_cycles;
  start_us_ = NowMicros();
  writer_ = std::thread([this] { WriterLoop(); });
  active_.store(true, std::memory_order_release);
}

void Timeline::Shutdown() {
  bool was_active = active_.exchange(false);
  if (was_active) {
    {
      std::lock_guard<std::mutex> l(q_mu_);
      stop_ = true;
    }
    q_cv_.notify_all();
  }
  if (writer_.joinable()) writer_.join();
}

void Timeline::Emit(char phase, const std::string& tensor,
                    const std::string& name, const std::string& args, int64_t abs_us) {
  Record r{phase, tensor, name, args, (abs_us >= 0 ? abs_us : NowMicros()) - start_us_};
  {
    std::lock_guard<std::mutex> l(q_mu_);
    queue_.push_back(std::move(r));
  }
  q_cv_.notify_one();
}

void Timeline::NegotiateStart(const std::string& tensor, Request::Type type) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    State& s = states_[tensor];
    if (s != State::UNKNOWN) return;  // already negotiating
    s = State::NEGOTIATING;
  }
  Emit('B', tensor, std::string("NEGOTIATE_") + Request::TypeName(type));
}

void Timeline::NegotiateRankReady(const std::string& tensor, int rank) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    if (states_[tensor] != State::NEGOTIATING) return;
  }
  Emit('X', tensor, std::to_string(rank));
}

void Timeline::NegotiateEnd(const std::string& tensor) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    auto it = states_.find(tensor);
    if (it == states_.end() || it->second != State::NEGOTIATING) return;
    it->second = State::UNKNOWN;
  }
  Emit('E', tensor, "");
}

void Timeline::Start(const std::string& tensor, Response::Type type,
                     int64_t size_bytes) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    State& s = states_[tensor];
    if (s == State::NEGOTIATING) {
      // Cached tensors skip negotiation on non-coordinator paths; close any
      // stale span so B/E stay balanced.
      s = State::UNKNOWN;
      Emit('E', tensor, "");
    }
    if (s != State::UNKNOWN) return;
    s = State::TOP_LEVEL;
  }
  std::string args;
  if (size_bytes > 0) args = "\"bytes\": " + std::to_string(size_bytes);
  Emit('B', tensor, Response::TypeName(type), args);
  NvtxPush(false, tensor, Response::TypeName(type));
}

void Timeline::ActivityStart(const std::string& tensor,
                             const std::string& activity) {
  ActivityStartAt(tensor, activity, -1);
}

void Timeline::ActivityStartAt(const std::string& tensor, const std::string& activity,
                               int64_t abs_us) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    auto it = states_.find(tensor);
    if (it == states_.end() || it->second != State::TOP_LEVEL) return;
    it->second = State::ACTIVITY;
  }
  Emit('B', tensor, activity, "", abs_us);
  NvtxPush(true, tensor, activity);
}

void Timeline::ActivityEnd(const std::string& tensor) { ActivityEndAt(tensor, -1); }

void Timeline::ActivityEndAt(const std::string& tensor, int64_t abs_us) {
  if (!Initialized()) return;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    auto it = states_.find(tensor);
    if (it == states_.end() || it->second != State::ACTIVITY) return;
    it->second = State::TOP_LEVEL;
  }
  Emit('E', tensor, "", "", abs_us);
  NvtxPop(true, tensor);
}

void Timeline::ActivityStartAll(const std::vector<TensorTableEntry>& entries,
                                const std::string& activity) {
  if (!Initialized()) return;
  for (auto& e : entries) ActivityStart(e.name, activity);
}

void Timeline::ActivityEndAll(const std::vector<TensorTableEntry>& entries) {
  if (!Initialized()) return;
  for (auto& e : entries) ActivityEnd(e.name);
}

void Timeline::End(const std::string& tensor) { EndAt(tensor, -1); }

void Timeline::EndAt(const std::string& tensor, int64_t abs_us) {
  if (!Initialized()) return;
  bool close_activity = false;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    auto it = states_.find(tensor);
    if (it == states_.end()) return;
    if (it->second == State::ACTIVITY) close_activity = true;
    else if (it->second != State::TOP_LEVEL) return;
    states_.erase(it);
  }
  if (close_activity) {
    Emit('E', tensor, "", "", abs_us);
    NvtxPop(true, tensor);
  }
  Emit('E', tensor, "", "", abs_us);
  NvtxPop(false, tensor);
}

void Timeline::NvtxPush(bool activity, const std::string& tensor, const std::string& name) {
  const uint64_t id = NvtxTimelineRangeStart(activity, tensor, name);
  if (id == 0) return;
  std::lock_guard<std::mutex> l(state_mu_);
  auto& open = activity ? nvtx_activities_ : nvtx_ops_;
  auto it = open.find(tensor);
  if (it != open.end()) NvtxTimelineRangeEnd(activity, it->second);
  open[tensor] = id;
}

void Timeline::NvtxPop(bool activity, const std::string& tensor) {
  uint64_t id = 0;
  {
    std::lock_guard<std::mutex> l(state_mu_);
    auto& open = activity ? nvtx_activities_ : nvtx_ops_;
    auto it = open.find(tensor);
    if (it == open.end()) return;
    id = it->second;
    open.erase(it);
  }
  NvtxTimelineRangeEnd(activity, id);
}

void Timeline::MarkCycleStart() {
  if (!Initialized() || !mark_cycles_) return;
  Emit('i', "", "CYCLE_START");
}

void Timeline::WriterLoop() {
  std::vector<Record> batch;
  for (;;) {
    {
      std::unique_lock<std::mutex> l(q_mu_);
      q_cv_.wait(l, [this] { return stop_ || !queue_.empty(); });
      batch.swap(queue_);
      if (batch.empty() && stop_) break;
    }
    for (auto& r : batch) WriteRecord(r);
    batch.clear();
    std::fflush(file_);
  }
  std::fputs("\n]\n", file_);
  std::fclose(file_);
  file_ = nullptr;
}

void Timeline::WriteRecord(const Record& r) {
  int pid = 0;
  if (!r.tensor.empty()) {
    auto it = tensor_pid_.find(r.tensor);
    if (it == tensor_pid_.end()) {
      pid = static_cast<int>(tensor_pid_.size()) + 1;
      tensor_pid_.emplace(r.tensor, pid);
      std::fprintf(file_,
                   "%s{\"name\": \"process_name\", \"ph\": \"M\", \"pid\": %d, "
                   "\"args\": {\"name\": \"%s\"}},\n"
                   "{\"name\": \"process_sort_index\", \"ph\": \"M\", \"pid\": "
                   "%d, \"args\": {\"sort_index\": %d}}",
                   first_event_ ? "" : ",\n", pid,
                   JsonEscape(r.tensor).c_str(), pid, pid);
      first_event_ = false;
    } else {
      pid = it->second;
    }
  }
  std::fprintf(file_, "%s{\"ph\": \"%c\"", first_event_ ? "" : ",\n", r.phase);
  first_event_ = false;
  if (r.phase != 'E')
    std::fprintf(file_, ", \"name\": \"%s\"", JsonEscape(r.name).c_str());
  std::fprintf(file_, ", \"ts\": %lld, \"pid\": %d",
               static_cast<long long>(r.ts_us), pid);
  if (r.phase == 'X') std::fputs(", \"dur\": 0", file_);
  if (r.phase == 'i') std::fputs(", \"s\": \"g\"", file_);
  if (!r.args.empty()) std::fprintf(file_, ", \"args\": {%s}", r.args.c_str());
  std::fputs("}", file_);
}

}  // namespace hvd
