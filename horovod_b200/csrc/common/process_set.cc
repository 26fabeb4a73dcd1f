#include "process_set.h"

#include <algorithm>
#include <stdexcept>

namespace hvd {

void ProcessSetTable::Initialize(TcpMesh* mesh, Timeline* timeline,
                                 ParameterManager* params,
                                 const ControllerOptions& opts,
                                 bool stall_check, int stall_warn_s,
                                 int stall_shutdown_s) {
  std::lock_guard<std::recursive_mutex> l(mu_);
  mesh_ = mesh;
  timeline_ = timeline;
  params_ = params;
  opts_ = opts;
  stall_check_ = stall_check;
  stall_warn_s_ = stall_warn_s;
  stall_shutdown_s_ = stall_shutdown_s;
  sets_.clear();
  next_id_ = 0;
  std::vector<int> all(mesh->size());
  for (int i = 0; i < mesh->size(); ++i) all[i] = i;
  RegisterProcessSet(std::move(all));
}

void ProcessSetTable::Clear() {
  std::lock_guard<std::recursive_mutex> l(mu_);
  sets_.clear();
  next_id_ = 0;
}

int32_t ProcessSetTable::RegisterProcessSet(std::vector<int> ranks) {
  std::lock_guard<std::recursive_mutex> l(mu_);
  std::sort(ranks.begin(), ranks.end());
  ranks.erase(std::unique(ranks.begin(), ranks.end()), ranks.end());
  if (ranks.empty()) throw std::invalid_argument("hvd: empty process set");
  for (int r : ranks)
    if (r < 0 || r >= mesh_->size())
      throw std::invalid_argument("hvd: process set rank out of range");
  int32_t existing = FindId(ranks);
  if (existing >= 0) return existing;
  int32_t id = next_id_++;
  std::unique_ptr<ProcessSet> ps(
      new ProcessSet(id, mesh_, std::move(ranks), *timeline_, *params_));
  ps->controller.options() = opts_;
  ps->response_cache.set_capacity(opts_.cache_capacity);
  ps->controller.stall_inspector().SetPerformStallCheck(stall_check_);
  ps->controller.stall_inspector().SetStallWarningTimeSeconds(stall_warn_s_);
  ps->controller.stall_inspector().SetStallShutdownTimeSeconds(stall_shutdown_s_);
  sets_[id] = std::move(ps);
  return id;
}

void ProcessSetTable::DeregisterProcessSet(int32_t id) {
  std::lock_guard<std::recursive_mutex> l(mu_);
  if (id == 0) throw std::invalid_argument("hvd: cannot remove the global process set");
  auto it = sets_.find(id);
  if (it == sets_.end()) return;
  it->second->tensor_queue.FinalizeTensorQueue(
      Status::Aborted("Process set has been removed."));
  sets_.erase(it);
}

bool ProcessSetTable::Contains(int32_t id) const {
  std::lock_guard<std::recursive_mutex> l(mu_);
  return sets_.count(id) != 0;
}

ProcessSet& ProcessSetTable::Get(int32_t id) {
  std::lock_guard<std::recursive_mutex> l(mu_);
  auto it = sets_.find(id);
  if (it == sets_.end())
    throw std::out_of_range("hvd: unknown process set id " + std::to_string(id));
  return *it->second;
}

std::vector<int32_t> ProcessSetTable::Ids() const {
  std::lock_guard<std::recursive_mutex> l(mu_);
  std::vector<int32_t> ids;
  for (auto& kv : sets_) ids.push_back(kv.first);
  return ids;
}

int32_t ProcessSetTable::FindId(const std::vector<int>& ranks) const {
  std::lock_guard<std::recursive_mutex> l(mu_);
  for (auto& kv : sets_)
    if (kv.second->ranks() == ranks) return kv.first;
  return -1;
}

}  // namespace hvd
