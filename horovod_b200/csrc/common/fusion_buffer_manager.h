// Persistent fusion buffers: one per (device, stream slot), kept between
// collectives and re-allocated only when the fusion threshold has changed
// (the autotuner moves it) or a larger buffer is needed. The memory itself
// comes from the caller's allocator (host vector, cudaMalloc), so the manager
// only owns the policy.
//
// Parity: horovod/common/fusion_buffer_manager.cc:21-50.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <utility>

namespace hvd {

class FusionBufferManager {
public:
  using Alloc = std::function<void*(size_t bytes)>;
  using Free = std::function<void(void* ptr)>;

  FusionBufferManager() = default;
  FusionBufferManager(Alloc alloc, Free free) : alloc_(std::move(alloc)), free_(std::move(free)) {}
  ~FusionBufferManager() { Clear(); }
  FusionBufferManager(const FusionBufferManager&) = delete;
  FusionBufferManager& operator=(const FusionBufferManager&) = delete;

  // Buffer of at least `needed` bytes for (device, slot). `threshold` is the
  // fusion threshold in effect: the buffer is sized for it (or for `needed`
  // if that is larger) and replaced when the threshold differs from the one
  // it was made for. `before_free` runs before an old buffer is released
  // (e.g. a stream synchronisation).
  void* Get(int device, int slot, size_t needed, size_t threshold,
            const std::function<void()>& before_free = nullptr);
  size_t SizeOf(int device, int slot) const;
  int reallocations() const { return reallocations_; }
  void Clear();

private:
  struct Buffer {
    void* ptr = nullptr;
    size_t bytes = 0;
    size_t threshold = 0;
  };
  Alloc alloc_;
  Free free_;
  std::map<std::pair<int, int>, Buffer> buffers_;
  int reallocations_ = 0;
};

}  // namespace hvd
