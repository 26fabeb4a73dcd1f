// Symmetric device memory shared by the ranks of one node.
//
// Every rank allocates the same-sized buffer with the CUDA virtual memory
// API, exports it as a POSIX file descriptor, passes the descriptor to its
// peers over Unix-domain sockets and maps every peer's buffer into its own
// address space, so kernels can load from and store to any rank's buffer
// over NVLink with plain pointers. When the GPUs support NVLink multicast
// the buffers are additionally bound to one multicast object, whose mapping
// lets `multimem` instructions reduce across / broadcast to all ranks inside
// the NVSwitch.
//
// The reference has no counterpart (its GPU data plane is NCCL only,
// horovod/common/ops/nccl_operations.cc); this is the foundation of the
// in-kernel collectives here.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../common/common.h"
#include "../transport/mesh.h"

namespace hvd {

constexpr int SYMM_MAX_RANKS = 8;
// Flag slots per source rank in the signal pad (one per CTA of a kernel).
constexpr int SYMM_MAX_BLOCKS = 512;
// Flag banks of MAX_RANKS x MAX_BLOCKS words each. Bank 0 holds the barrier
// flags of every kernel (kernels of one process set run one after the other
// on one stream and share an epoch counter); bank 1 is the token mailbox of
// the kernels that address symmetric-heap tensors by offset; banks 2 and 3
// are spare.
constexpr int SYMM_FLAG_BANKS = 4;
// Each process set gets its own copy of the banks (slot = set id modulo
// this), so epochs of different sets never meet in one flag word.
constexpr int SYMM_FLAG_SETS = 8;

struct SymmArenaInfo {
  int rank = 0;
  int world = 1;
  int device = 0;
  size_t data_bytes = 0;    // usable staging bytes per rank
  size_t signal_bytes = 0;  // flag pad bytes per rank
  bool multicast = false;
  void* local = nullptr;
  void* peers[SYMM_MAX_RANKS] = {};      // data base of every rank
  void* mc = nullptr;                    // multicast view of the data
  uint32_t* flags[SYMM_MAX_RANKS] = {};  // signal pad of every rank
  uint32_t* mc_flags = nullptr;          // multicast view of the signal pad
};

class SymmArena {
public:
  SymmArena() = default;
  ~SymmArena() { Destroy(); }
  SymmArena(const SymmArena&) = delete;
  SymmArena& operator=(const SymmArena&) = delete;

  // Collective over `comm` (all ranks must be on this node and pass the same
  // sizes). `device` is this rank's CUDA device. Returns an error status
  // (never throws) when the platform cannot provide peer-mapped memory; the
  // caller then falls back to NCCL. `token` makes socket names unique per
  // job and per (re)initialisation.
  Status Create(Comm& comm, int device, size_t data_bytes, bool want_multicast,
                uint64_t token);
  void Destroy();

  bool valid() const { return info_.local != nullptr; }
  const SymmArenaInfo& info() const { return info_; }

private:
  SymmArenaInfo info_;
  size_t total_bytes_ = 0;  // mapped bytes per rank (data + signal, rounded)
  std::vector<unsigned long long> handles_;  // CUmemGenericAllocationHandle
  std::vector<unsigned long long> vas_;      // CUdeviceptr per rank
  unsigned long long mc_handle_ = 0;
  unsigned long long mc_va_ = 0;
  bool mc_bound_ = false;
};

}  // namespace hvd
