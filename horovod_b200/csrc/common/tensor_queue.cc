#include "tensor_queue.h"

#include <stdexcept>

namespace hvd {

Status TensorQueue::AddToTensorQueueMulti(std::vector<TensorTableEntry>& entries,
                                          std::vector<Request>& requests) {
  std::lock_guard<std::mutex> l(mu_);
  for (auto& e : entries) {
    if (table_.count(e.name)) return Status::InvalidArgument(DUPLICATE_NAME_ERROR_MESSAGE);
  }
  // Names inside one call must be distinct too.
  for (size_t i = 0; i < entries.size(); ++i)
    for (size_t j = i + 1; j < entries.size(); ++j)
      if (entries[i].name == entries[j].name)
        return Status::InvalidArgument(DUPLICATE_NAME_ERROR_MESSAGE);
  for (size_t i = 0; i < entries.size(); ++i) {
    std::string name = entries[i].name;
    table_.emplace(std::move(name), std::move(entries[i]));
    queue_.push_back(std::move(requests[i]));
  }
  return Status::OK();
}

Status TensorQueue::AddToTensorQueue(TensorTableEntry entry, Request request) {
  std::vector<TensorTableEntry> es;
  std::vector<Request> rs;
  es.push_back(std::move(entry));
  rs.push_back(std::move(request));
  return AddToTensorQueueMulti(es, rs);
}

void TensorQueue::PopMessagesFromQueue(std::deque<Request>& out) {
  std::lock_guard<std::mutex> l(mu_);
  while (!queue_.empty()) {
    out.push_back(std::move(queue_.front()));
    queue_.pop_front();
  }
}

void TensorQueue::PushMessagesToQueue(std::deque<Request>& requests) {
  std::lock_guard<std::mutex> l(mu_);
  while (!requests.empty()) {
    queue_.push_front(std::move(requests.back()));
    requests.pop_back();
  }
}

void TensorQueue::GetTensorEntriesFromResponse(
    const Response& response, std::vector<TensorTableEntry>& entries,
    bool joined) {
  std::lock_guard<std::mutex> l(mu_);
  entries.reserve(response.names.size());
  for (size_t i = 0; i < response.names.size(); ++i) {
    const std::string& name = response.names[i];
    auto it = table_.find(name);
    if (it != table_.end()) {
      entries.push_back(std::move(it->second));
      table_.erase(it);
      continue;
    }
    // A joined rank sees the others' error responses too (for example an
    // allgather refused because of the join); it has nothing to fail.
    if (joined && response.type == Response::ERROR) continue;
    if (!joined)
      throw std::logic_error("hvd: response names tensor '" + name +
                             "' that this rank never enqueued");
    // Joined rank: stand-in that contributes zeros and discards the result.
    TensorTableEntry e;
    e.name = name;
    e.dtype = response.dtype;
    e.wire_dtype = response.wire_dtype;
    e.reduce_op = response.reduce_op;
    e.prescale = response.prescale;
    e.postscale = response.postscale;
    e.device = response.devices.empty() ? CPU_DEVICE_ID : response.devices[0];
    if (i < response.tensor_sizes.size())
      e.shape = TensorShape({response.tensor_sizes[i]});
    entries.push_back(std::move(e));
  }
}

TensorTableEntry TensorQueue::GetTensorEntry(const std::string& name) const {
  std::lock_guard<std::mutex> l(mu_);
  auto it = table_.find(name);
  if (it == table_.end())
    throw std::logic_error("hvd: no pending tensor named '" + name + "'");
  TensorTableEntry meta;
  meta.name = it->second.name;
  meta.shape = it->second.shape;
  meta.dtype = it->second.dtype;
  meta.device = it->second.device;
  meta.root_rank = it->second.root_rank;
  meta.reduce_op = it->second.reduce_op;
  meta.prescale = it->second.prescale;
  meta.postscale = it->second.postscale;
  meta.group_id = it->second.group_id;
  return meta;
}

bool TensorQueue::IsTensorPresentInTable(const std::string& name) const {
  std::lock_guard<std::mutex> l(mu_);
  return table_.count(name) != 0;
}

bool TensorQueue::PopJoinEntry(TensorTableEntry* out) {
  std::lock_guard<std::mutex> l(mu_);
  auto it = table_.find(JOIN_TENSOR_NAME);
  if (it == table_.end()) return false;
  *out = std::move(it->second);
  table_.erase(it);
  return true;
}

void TensorQueue::FinalizeTensorQueue(const Status& status) {
  std::unordered_map<std::string, TensorTableEntry> drained;
  {
    std::lock_guard<std::mutex> l(mu_);
    drained.swap(table_);
    queue_.clear();
  }
  for (auto& kv : drained) kv.second.Finish(status);
}

int64_t TensorQueue::GetTensorDataForAutotuner(
    const ResponseList& responses, std::vector<std::string>& names) const {
  std::lock_guard<std::mutex> l(mu_);
  int64_t total = 0;
  for (auto& r : responses.responses) {
    if (r.type == Response::ERROR || r.type == Response::JOIN) continue;
    for (auto& n : r.names) {
      auto it = table_.find(n);
      if (it == table_.end()) continue;
      names.push_back(n);
      total += it->second.size_bytes();
    }
  }
  return total;
}

size_t TensorQueue::pending() const {
  std::lock_guard<std::mutex> l(mu_);
  return table_.size();
}

}  // namespace hvd
