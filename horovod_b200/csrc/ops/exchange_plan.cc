#include "exchange_plan.h"

#include <algorithm>
#include <stdexcept>

#include "../kernels/kernels.h"

namespace hvd {

namespace {
constexpr int64_t STAGING_ALIGN = 256;
int64_t RoundUpTo(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
}  // namespace

void PlanExchangeRounds(std::vector<ExchangeBlock>& blocks, int rank, int world,
                        int64_t region_bytes, bool push, const ExchangeRoundFn& launch) {
  const int64_t cap = region_bytes;
  const int me = rank;
  // When the staged data of a source (pulling) or of everybody (pushing) does
  // not fit the region, every block is cut into the same number of slices and
  // the rounds go slice by slice: round k moves slice k of every block, so
  // every rank is busy in every round and all NVLink links stay in use.
  // Pulling fills the source's region; pushing fills the receiver's region
  // (every region, for a block that goes to everybody).
  std::vector<int64_t> staged(world, 0);
  for (auto& b : blocks) {
    const bool remote = world > 1 && (b.dst_rank < 0 || b.dst_rank != b.src_rank);
    if (!remote) continue;
    const int64_t need = RoundUpTo(b.bytes, STAGING_ALIGN) + STAGING_ALIGN;
    if (!push) {
      staged[b.src_rank] += need;
    } else if (b.dst_rank >= 0) {
      staged[b.dst_rank] += need;
    } else {
      for (auto& s : staged) s += need;
    }
  }
  const int64_t most = *std::max_element(staged.begin(), staged.end());
  const int64_t slices = std::max<int64_t>(1, (most + cap - 1) / cap);
  std::vector<ExchangeBlock> parts;
  for (int64_t k = 0; k < slices; ++k) {
    for (auto& b : blocks) {
      if (b.bytes == 0) continue;
      const int64_t per = RoundUpTo((b.bytes + slices - 1) / slices, STAGING_ALIGN);
      const int64_t pos = k * per;
      if (pos >= b.bytes) continue;
      ExchangeBlock p = b;
      p.src = b.src ? b.src + pos : nullptr;
      p.dst = b.dst ? b.dst + pos : nullptr;
      p.bytes = std::min(per, b.bytes - pos);
      parts.push_back(p);
    }
  }
  size_t next = 0;
  while (next < parts.size()) {
    std::vector<ExchangeStageSeg> stage;
    std::vector<ExchangePullSeg> pull;
    // One cursor per region. Pulling: a block sits in its source's region.
    // Pushing: in its receiver's region, or, when it goes to everybody, at
    // one offset that is free in every region.
    std::vector<int64_t> cursor(world, 0);
    size_t n = 0;
    int64_t round_bytes = 0;
    std::vector<ExchangeRoundBlock> round;
    while (next + n < parts.size() && n < 4096) {
      const ExchangeBlock& b = parts[next + n];
      const bool remote = world > 1 && (b.dst_rank < 0 || b.dst_rank != b.src_rank);
      const bool wanted = (b.dst_rank < 0 || b.dst_rank == me) && b.dst != nullptr;
      if (!remote) {
        // Data a rank keeps for itself: a local copy, no region space.
        if (b.src_rank == me && wanted) stage.push_back({b.src, b.dst, -1, b.bytes, -2});
      } else {
        const int64_t padded = RoundUpTo(b.bytes, STAGING_ALIGN);
        const bool everywhere = push && b.dst_rank < 0;
        const int region = push ? b.dst_rank : b.src_rank;
        const int64_t off = everywhere ? *std::max_element(cursor.begin(), cursor.end())
                                       : cursor[region];
        if (off + padded > cap) break;
        if (everywhere) {
          std::fill(cursor.begin(), cursor.end(), off + padded);
        } else {
          cursor[region] = off + padded;
        }
        if (b.src_rank == me) {
          stage.push_back({b.src, wanted ? b.dst : nullptr, off, b.bytes,
                           push ? b.dst_rank : -2});
        } else if (wanted) {
          pull.push_back({b.dst, off, b.bytes, push ? me : b.src_rank, b.src_rank,
                          static_cast<int32_t>(round.size())});
        }
        round.push_back({b.src_rank, b.bytes});
      }
      round_bytes += b.bytes;
      ++n;
    }
    if (n == 0) throw std::runtime_error("exchange block exceeds staging capacity");
    launch(stage, pull, round_bytes, round);
    next += n;
  }
}


ExchangeRoundSync ComputeExchangeRoundSync(const std::vector<ExchangeRoundBlock>& round,
                                           int world, int ctas, int64_t chunk_bytes) {
  ExchangeRoundSync out;
  std::vector<int64_t> published(world, 0);  // chunks per source so far
  out.before.assign(round.size(), 0);        // ... before each block
  for (size_t i = 0; i < round.size(); ++i) {
    const int src = round[i].src_rank;
    out.before[i] = published[src];
    published[src] += kern::ExchangeChunkCount(round[i].bytes, ctas, chunk_bytes);
  }
  const int64_t most = published.empty() ? 0 : *std::max_element(published.begin(), published.end());
  out.done_epochs = static_cast<uint32_t>(std::min<int64_t>(most + 1, int64_t(1) << 31));
  return out;
}

}  // namespace hvd
