// Host-side planning of the exchange kernel's work (allgather, broadcast,
// alltoall): from the global list of blocks (who owns which bytes, who wants
// them) to the rounds, region offsets and chunk counters of the launches.
// Everything here is deterministic in data that all ranks share, so the ranks
// agree on rounds and offsets without talking. No CUDA calls: usable by the
// executor and by tests alike.
#ifndef HVD_B200_EXCHANGE_PLAN_H
#define HVD_B200_EXCHANGE_PLAN_H

#include <cstdint>
#include <functional>
#include <vector>

namespace hvd {

struct ExchangeBlock {
  int src_rank;     // set rank that owns the data
  int dst_rank;     // receiving set rank, or -1 for everybody
  const char* src;  // valid on src_rank only
  char* dst;        // where this rank wants the data (null = not wanted)
  int64_t bytes;
};

// Segments handed to the exchange kernel (see kern::ExchangePlan).
struct ExchangeStageSeg {
  const void* src;
  void* self_dst;
  int64_t off;    // offset in the region, < 0 = local copy only
  int64_t bytes;
  int32_t dst;    // -2 own region, -1 every other rank's region, >= 0 that rank's region
};
struct ExchangePullSeg {
  void* dst;
  int64_t off;
  int64_t bytes;
  int32_t src_rank;  // set rank whose region holds the data
  int32_t sig_rank;  // set rank whose progress counter announces it
  int32_t block;     // index into the round's block list
};
// Every staged block of one exchange round, in the order all ranks process
// them (what the chunk counters of the kernel are derived from).
struct ExchangeRoundBlock {
  int32_t src_rank;
  int64_t bytes;
};

using ExchangeRoundFn =
    std::function<void(const std::vector<ExchangeStageSeg>&, const std::vector<ExchangePullSeg>&,
                       int64_t round_bytes, const std::vector<ExchangeRoundBlock>&)>;

// Calls `launch` once per round with rank `rank`'s segments. A block that
// somebody else needs is staged in a region of `region_bytes`: the source's
// own region when pulling, the receiver's region when pushing (a block for
// everybody takes one offset that is free in every region). When the data
// does not fit a region, every block is cut into the same number of slices
// and the rounds go slice by slice.
void PlanExchangeRounds(std::vector<ExchangeBlock>& blocks, int rank, int world,
                        int64_t region_bytes, bool push, const ExchangeRoundFn& launch);

// Chunk counters of one round: how many chunks a source has published before
// each of its blocks, and the epochs the launch consumes (the largest chunk
// total of any rank, plus one for a final barrier).
struct ExchangeRoundSync {
  std::vector<int64_t> before;
  uint32_t done_epochs;
};
ExchangeRoundSync ComputeExchangeRoundSync(const std::vector<ExchangeRoundBlock>& round,
                                           int world, int ctas, int64_t chunk_bytes);

}  // namespace hvd

#endif
