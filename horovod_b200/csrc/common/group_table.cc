#include "group_table.h"

namespace hvd {

int32_t GroupTable::RegisterGroup(std::vector<std::string> names) {
  std::lock_guard<std::mutex> l(mu_);
  int32_t id;
  if (!free_ids_.empty()) {
    id = free_ids_.front();
    free_ids_.pop();
  } else {
    id = next_id_++;
  }
  for (auto& n : names) name_to_id_[n] = id;
  id_to_names_[id] = std::move(names);
  return id;
}

void GroupTable::DeregisterGroups(const std::vector<std::string>& names) {
  std::lock_guard<std::mutex> l(mu_);
  for (auto& n : names) {
    auto it = name_to_id_.find(n);
    if (it == name_to_id_.end()) continue;
    int32_t id = it->second;
    auto git = id_to_names_.find(id);
    if (git != id_to_names_.end()) {
      for (auto& member : git->second) name_to_id_.erase(member);
      id_to_names_.erase(git);
      free_ids_.push(id);
    }
  }
}

int32_t GroupTable::GetGroupIDFromTensorName(const std::string& name) const {
  std::lock_guard<std::mutex> l(mu_);
  auto it = name_to_id_.find(name);
  return it == name_to_id_.end() ? NULL_GROUP_ID : it->second;
}

std::vector<std::string> GroupTable::GetGroupTensorNames(int32_t id) const {
  std::lock_guard<std::mutex> l(mu_);
  auto it = id_to_names_.find(id);
  return it == id_to_names_.end() ? std::vector<std::string>() : it->second;
}

bool GroupTable::empty() const {
  std::lock_guard<std::mutex> l(mu_);
  return id_to_names_.empty();
}

}  // namespace hvd
