// Cache of negotiated single-tensor responses with stable bit positions, and
// the per-cycle coordinator that agrees across ranks on which cached
// responses are ready using one bit-vector allreduce.
//
// Parity: horovod/common/response_cache.h:45-169, response_cache.cc:69-498.
// Every rank applies the same put/get/erase sequence, so bit positions and
// LRU order stay identical everywhere without extra communication.
#pragma once

#include <cstdint>
#include <functional>
#include <list>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "message.h"

namespace hvd {

class TensorQueue;

class ResponseCache {
public:
  enum class CacheState { MISS = 0, HIT = 1, INVALID = 2 };

  void clear();
  void set_capacity(uint32_t capacity);
  uint32_t capacity() const { return capacity_; }
  size_t num_active_bits() const { return entries_.size(); }

  // Compares a new request against what was negotiated before under the
  // same name.
  CacheState cached(const Request& request) const;
  // Inserts (or refreshes) the single-tensor responses that make up
  // `response`. Shapes come from the tensor queue when this rank has the
  // tensor pending, otherwise from the response's element counts.
  void put(const Response& response, const TensorQueue& queue, bool joined);
  // Returns the response and marks it most recently used.
  const Response& get_response(uint32_t bit);
  const Response& peek_response(uint32_t bit) const;
  uint32_t peek_cache_bit(const std::string& name) const;
  bool has_name(const std::string& name) const {
    return name_to_bit_.count(name) != 0;
  }
  std::vector<uint32_t> list_all_bits() const;
  void erase_response(uint32_t bit);
  // Renumbers bits to follow LRU order after erasures/evictions.
  void update_cache_bits();

private:
  struct Params {
    DataType dtype;
    std::vector<int64_t> shape;
    bool shape_is_synthetic;  // built from an element count (joined rank)
    int32_t device;
    double prescale, postscale;
    ReduceOp reduce_op;
    int32_t root_rank;
    DataType wire_dtype;
  };
  struct Entry {
    Response response;
    Params params;
  };
  void put_one(Response response, Params params);

  uint32_t capacity_ = 0;
  std::list<Entry> lru_;  // front = most recently used
  std::vector<std::list<Entry>::iterator> entries_;  // indexed by bit
  std::unordered_map<std::string, uint32_t> name_to_bit_;
  bool bits_outdated_ = false;
};

// One cycle's view of cache hits and global flags, synchronised with a
// bitwise AND (and, if anything was invalidated, a bitwise OR) across ranks.
class CacheCoordinator {
public:
  explicit CacheCoordinator(size_t num_active_bits)
      : num_active_bits_(num_active_bits) {}

  void record_hit(uint32_t bit) { hits_.insert(bit); }
  void erase_hit(uint32_t bit) { hits_.erase(bit); }
  void record_invalid_bit(uint32_t bit) {
    invalid_bits_.insert(bit);
    invalid_in_queue_ = true;
  }
  void set_should_shut_down(bool v) { should_shut_down_ = v; }
  void set_uncached_in_queue(bool v) { uncached_in_queue_ = v; }

  const std::set<uint32_t>& cache_hits() const { return hits_; }
  const std::set<uint32_t>& invalid_bits() const { return invalid_bits_; }
  bool should_shut_down() const { return should_shut_down_; }
  bool uncached_in_queue() const { return uncached_in_queue_; }

  using BitAllreduce =
      std::function<void(uint64_t* words, size_t n, bool bitwise_and)>;
  // After sync(): cache_hits() holds only bits every rank hit,
  // invalid_bits() holds bits any rank invalidated, and the flags are the
  // logical OR over ranks.
  void sync(const BitAllreduce& allreduce);

private:
  enum StatusBit { SHOULD_SHUT_DOWN = 0, UNCACHED_IN_QUEUE = 1,
                   INVALID_IN_QUEUE = 2, NUM_STATUS_BITS = 3 };
  size_t num_active_bits_;
  std::set<uint32_t> hits_;
  std::set<uint32_t> invalid_bits_;
  bool should_shut_down_ = false;
  bool uncached_in_queue_ = false;
  bool invalid_in_queue_ = false;
};

}  // namespace hvd
