// Hand-off point between framework threads (which enqueue collectives) and
// the background thread (which negotiates and executes them): a table of
// pending entries keyed by tensor name plus a FIFO of their requests.
//
// Parity: horovod/common/tensor_queue.h:28-64, tensor_queue.cc:27-183.
// Difference: a rank that has joined does not allocate zero tensors; it
// fabricates entries with null input/output pointers, which every op treats
// as "contribute zeros, discard the result".
#pragma once

#include <deque>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "message.h"

namespace hvd {

constexpr const char* JOIN_TENSOR_NAME = "join.noname";

class TensorQueue {
public:
  // All-or-nothing: if any name is already pending nothing is added and
  // DUPLICATE_NAME_ERROR is returned.
  Status AddToTensorQueueMulti(std::vector<TensorTableEntry>& entries,
                               std::vector<Request>& requests);
  Status AddToTensorQueue(TensorTableEntry entry, Request request);

  void PopMessagesFromQueue(std::deque<Request>& out);
  // Returns requests to the front of the FIFO, to be retried next cycle.
  void PushMessagesToQueue(std::deque<Request>& requests);

  // Moves the entries named by `response` out of the table. When `joined`
  // is set, names this rank never enqueued become zero-contribution entries.
  void GetTensorEntriesFromResponse(const Response& response,
                                    std::vector<TensorTableEntry>& entries,
                                    bool joined);
  // Copy of a pending entry's metadata (throws if absent).
  TensorTableEntry GetTensorEntry(const std::string& name) const;
  bool IsTensorPresentInTable(const std::string& name) const;
  // Takes the join entry out (if this rank joined) and returns it.
  bool PopJoinEntry(TensorTableEntry* out);

  // Fails every pending entry with `status` (used at shutdown).
  void FinalizeTensorQueue(const Status& status);
  // Total payload bytes named by the responses (autotuner score numerator).
  int64_t GetTensorDataForAutotuner(const ResponseList& responses,
                                    std::vector<std::string>& names) const;
  size_t pending() const;

private:
  mutable std::mutex mu_;
  std::unordered_map<std::string, TensorTableEntry> table_;
  std::deque<Request> queue_;
};

}  // namespace hvd
