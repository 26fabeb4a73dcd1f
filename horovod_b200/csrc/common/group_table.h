// Registry of grouped collectives: which tensor names must be negotiated and
// fused together. Ids are recycled after the group completes.
//
// Parity: horovod/common/group_table.cc:23-82.
#pragma once

#include <mutex>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

namespace hvd {

constexpr int32_t NULL_GROUP_ID = -1;

class GroupTable {
public:
  int32_t RegisterGroup(std::vector<std::string> names);
  void DeregisterGroups(const std::vector<std::string>& names);
  int32_t GetGroupIDFromTensorName(const std::string& name) const;
  std::vector<std::string> GetGroupTensorNames(int32_t id) const;
  bool empty() const;

private:
  mutable std::mutex mu_;
  std::unordered_map<std::string, int32_t> name_to_id_;
  std::unordered_map<int32_t, std::vector<std::string>> id_to_names_;
  std::queue<int32_t> free_ids_;
  int32_t next_id_ = 0;
};

}  // namespace hvd
