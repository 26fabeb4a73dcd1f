#include "fusion_buffer_manager.h"

#include <algorithm>

namespace hvd {

void* FusionBufferManager::Get(int device, int slot, size_t needed, size_t threshold,
                               const std::function<void()>& before_free) {
  Buffer& b = buffers_[{device, slot}];
  const size_t want = std::max(needed, threshold);
  if (b.ptr != nullptr && b.bytes >= needed && b.threshold == threshold) return b.ptr;
  if (b.ptr != nullptr && b.bytes >= want && b.threshold >= threshold &&
      b.bytes <= 2 * std::max<size_t>(want, 1)) {
    // Still a sensible size for the new threshold: keep it.
    b.threshold = threshold;
    return b.ptr;
  }
  if (b.ptr != nullptr) {
    if (before_free) before_free();
    free_(b.ptr);
    b = Buffer();
  }
  b.ptr = alloc_(want);
  b.bytes = b.ptr != nullptr ? want : 0;
  b.threshold = threshold;
  ++reallocations_;
  return b.ptr;
}

size_t FusionBufferManager::SizeOf(int device, int slot) const {
  auto it = buffers_.find({device, slot});
  return it == buffers_.end() ? 0 : it->second.bytes;
}

void FusionBufferManager::Clear() {
  for (auto& kv : buffers_)
    if (kv.second.ptr != nullptr && free_) free_(kv.second.ptr);
  buffers_.clear();
}

}  // namespace hvd
