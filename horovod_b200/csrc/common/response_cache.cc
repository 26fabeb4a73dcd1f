#include "response_cache.h"

#include <stdexcept>

#include "tensor_queue.h"

namespace hvd {

void ResponseCache::clear() {
  lru_.clear();
  entries_.clear();
  name_to_bit_.clear();
  bits_outdated_ = false;
}

void ResponseCache::set_capacity(uint32_t capacity) {
  if (capacity == capacity_) return;
  capacity_ = capacity;
  clear();
}

ResponseCache::CacheState ResponseCache::cached(const Request& q) const {
  auto it = name_to_bit_.find(q.name);
  if (it == name_to_bit_.end()) return CacheState::MISS;
  const Entry& e = *entries_[it->second];
  const Params& p = e.params;
  bool same_type =
      static_cast<int>(e.response.type) == static_cast<int>(q.type);
  bool same_shape;
  if (p.shape_is_synthetic) {
    int64_t n = 1;
    for (auto d : q.shape) n *= d;
    int64_t m = 1;
    for (auto d : p.shape) m *= d;
    same_shape = n == m;
  } else {
    same_shape = p.shape == q.shape;
  }
  bool same = same_type && p.dtype == q.dtype && same_shape &&
              p.device == q.device && p.prescale == q.prescale &&
              p.postscale == q.postscale && p.reduce_op == q.reduce_op &&
              (q.type != Request::ALLREDUCE || p.wire_dtype == q.wire_dtype) &&
              ((q.type != Request::BROADCAST && q.type != Request::ALLTOALL) ||
               p.root_rank == q.root_rank);  // alltoall: "even split" flag
  return same ? CacheState::HIT : CacheState::INVALID;
}

void ResponseCache::put_one(Response response, Params params) {
  const std::string name = response.names[0];
  auto it = name_to_bit_.find(name);
  if (it != name_to_bit_.end()) {
    // Refresh in place, keep the bit, move to the front.
    auto node = entries_[it->second];
    node->response = std::move(response);
    node->params = std::move(params);
    lru_.splice(lru_.begin(), lru_, node);
    bits_outdated_ = true;
    return;
  }
  uint32_t bit;
  if (lru_.size() >= capacity_) {
    // Evict the least recently used entry and take over its bit.
    auto victim = std::prev(lru_.end());
    bit = name_to_bit_.at(victim->response.names[0]);
    name_to_bit_.erase(victim->response.names[0]);
    lru_.erase(victim);
  } else {
    bit = static_cast<uint32_t>(entries_.size());
    entries_.emplace_back();
  }
  lru_.push_front(Entry{std::move(response), std::move(params)});
  entries_[bit] = lru_.begin();
  name_to_bit_[name] = bit;
  bits_outdated_ = true;
}

void ResponseCache::put(const Response& response, const TensorQueue& queue,
                        bool joined) {
  if (capacity_ == 0) return;
  size_t n = response.names.size();
  // ALLGATHER responses carry (size) dim-0 entries per tensor.
  size_t per_tensor = n ? response.tensor_sizes.size() / n : 0;
  for (size_t i = 0; i < n; ++i) {
    Response single;
    single.type = response.type;
    single.names.push_back(response.names[i]);
    single.devices = response.devices;
    single.dtype = response.dtype;
    single.reduce_op = response.reduce_op;
    single.prescale = response.prescale;
    single.postscale = response.postscale;
    single.wire_dtype = response.wire_dtype;
    single.root_rank = response.root_rank;
    for (size_t k = 0; k < per_tensor; ++k)
      single.tensor_sizes.push_back(response.tensor_sizes[i * per_tensor + k]);

    Params p;
    p.dtype = response.dtype;
    p.prescale = response.prescale;
    p.postscale = response.postscale;
    p.reduce_op = response.reduce_op;
    p.wire_dtype = response.wire_dtype;
    p.root_rank = 0;
    p.device = response.devices.empty() ? CPU_DEVICE_ID : response.devices[0];
    p.shape_is_synthetic = true;
    if (queue.IsTensorPresentInTable(response.names[i])) {
      TensorTableEntry meta = queue.GetTensorEntry(response.names[i]);
      p.shape = meta.shape.to_vector();
      p.device = meta.device;
      p.root_rank = meta.root_rank;
      p.shape_is_synthetic = false;
    } else if (!joined) {
      throw std::logic_error("hvd cache: tensor '" + response.names[i] +
                             "' missing from the queue");
    } else if (per_tensor >= 1) {
      p.shape = {single.tensor_sizes[0]};
    }
    put_one(std::move(single), std::move(p));
  }
}

const Response& ResponseCache::get_response(uint32_t bit) {
  auto node = entries_.at(bit);
  if (node != lru_.begin()) {
    lru_.splice(lru_.begin(), lru_, node);
    bits_outdated_ = true;
  }
  return node->response;
}

const Response& ResponseCache::peek_response(uint32_t bit) const {
  return entries_.at(bit)->response;
}

uint32_t ResponseCache::peek_cache_bit(const std::string& name) const {
  return name_to_bit_.at(name);
}

std::vector<uint32_t> ResponseCache::list_all_bits() const {
  std::vector<uint32_t> bits;
  bits.reserve(name_to_bit_.size());
  for (auto& kv : name_to_bit_) bits.push_back(kv.second);
  return bits;
}

void ResponseCache::erase_response(uint32_t bit) {
  auto node = entries_.at(bit);
  name_to_bit_.erase(node->response.names[0]);
  lru_.erase(node);
  // Leave a hole; update_cache_bits() compacts.
  entries_[bit] = lru_.end();
  bits_outdated_ = true;
}

void ResponseCache::update_cache_bits() {
  if (!bits_outdated_) return;
  entries_.clear();
  entries_.reserve(lru_.size());
  // Bit i goes to the i-th least recently used entry, so long-lived
  // tensors keep low, stable positions.
  uint32_t bit = 0;
  for (auto it = lru_.rbegin(); it != lru_.rend(); ++it, ++bit) {
    name_to_bit_[it->response.names[0]] = bit;
  }
  entries_.resize(lru_.size());
  for (auto it = lru_.begin(); it != lru_.end(); ++it)
    entries_[name_to_bit_[it->response.names[0]]] = it;
  bits_outdated_ = false;
}

void CacheCoordinator::sync(const BitAllreduce& allreduce) {
  // Word layout: bit 0..2 are the inverted status flags (so that AND acts as
  // OR on them), followed by one bit per cache entry.
  size_t total_bits = NUM_STATUS_BITS + num_active_bits_;
  size_t words = (total_bits + 63) / 64;
  std::vector<uint64_t> v(words, 0);
  auto set_bit = [&v](size_t b) { v[b / 64] |= (1ull << (b % 64)); };
  auto test_bit = [&v](size_t b) { return (v[b / 64] >> (b % 64)) & 1ull; };
  if (!should_shut_down_) set_bit(SHOULD_SHUT_DOWN);
  if (!uncached_in_queue_) set_bit(UNCACHED_IN_QUEUE);
  if (!invalid_in_queue_) set_bit(INVALID_IN_QUEUE);
  for (auto b : hits_) set_bit(NUM_STATUS_BITS + b);

  allreduce(v.data(), words, true);

  should_shut_down_ = !test_bit(SHOULD_SHUT_DOWN);
  uncached_in_queue_ = !test_bit(UNCACHED_IN_QUEUE);
  invalid_in_queue_ = !test_bit(INVALID_IN_QUEUE);
  std::set<uint32_t> common;
  for (auto b : hits_)
    if (test_bit(NUM_STATUS_BITS + b)) common.insert(b);
  hits_.swap(common);

  if (invalid_in_queue_) {
    std::vector<uint64_t> inv((num_active_bits_ + 63) / 64 + 1, 0);
    for (auto b : invalid_bits_) inv[b / 64] |= (1ull << (b % 64));
    allreduce(inv.data(), inv.size(), false);
    invalid_bits_.clear();
    for (size_t b = 0; b < num_active_bits_; ++b)
      if ((inv[b / 64] >> (b % 64)) & 1ull)
        invalid_bits_.insert(static_cast<uint32_t>(b));
    // A bit invalid anywhere is no longer a hit anywhere.
    for (auto b : invalid_bits_) hits_.erase(b);
  }
}

}  // namespace hvd
