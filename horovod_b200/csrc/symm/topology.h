// What the GPUs of this box look like to the collectives: peer access and
// P2P attributes between every pair, NVLink link state (through NVML, loaded
// with dlopen, read-only queries), and NVLink multicast support. Collected
// when the symmetric arena is first needed and on request from Python
// (`hvd.topology()`).
//
// The reference has no counterpart: it leaves topology to NCCL.
#pragma once

#include <string>
#include <vector>

namespace hvd {

struct GpuTopology {
  int device_count = 0;
  std::vector<std::string> names;
  std::vector<int> sm_counts;
  std::vector<long long> memory_bytes;
  std::vector<int> multicast_supported;            // per device, -1 unknown
  std::vector<int> nvlink_active_links;            // per device, -1 unknown
  std::vector<std::vector<int>> peer_access;       // [i][j] can i map j's memory
  std::vector<std::vector<int>> native_atomics;    // [i][j]
  std::vector<std::vector<int>> performance_rank;  // [i][j], lower is better
  bool all_pairs_peer = false;

  std::string Summary() const;
};

GpuTopology DiscoverTopology();

}  // namespace hvd
