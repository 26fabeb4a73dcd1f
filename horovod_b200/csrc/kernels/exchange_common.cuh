// Helpers shared by the exchange kernels: how a segment is divided among the
// CTAs of a launch and the cooperative byte copy to local memory, one peer or
// all peers.
#pragma once

#include "device_utils.cuh"

namespace hvd {
namespace kern {
namespace exch {

constexpr int THREADS = 512;
constexpr int64_t SMALL_SEGMENT = 64 * 1024;

// Byte range of a segment that CTA b is responsible for.
__device__ __forceinline__ void my_range(int64_t staging_off, int64_t bytes,
                                         int b, int G, int64_t* lo, int64_t* hi) {
  if (bytes <= SMALL_SEGMENT) {
    const int owner = static_cast<int>((staging_off >> 8) % G);
    *lo = 0;
    *hi = owner == b ? bytes : 0;
    return;
  }
  int64_t chunk = (bytes + G - 1) / G;
  chunk = (chunk + 255) & ~int64_t(255);
  *lo = min(bytes, b * chunk);
  *hi = min(bytes, *lo + chunk);
}

enum Target { TO_PEER, TO_ALL_MC, TO_ALL_LOOP, LOCAL_COPY };

// Cooperative copy of [lo, hi) bytes. dst_base/dst_all select the target.
__device__ __forceinline__ void copy_bytes(const char* src, char* dst,
                                           int64_t n, Target target,
                                           const SymmCtx& ctx,
                                           int64_t staging_off) {
  if (n <= 0) return;
  // `dst` is the local-view address; for TO_ALL_* the same offset is used in
  // every rank's buffer.
  const bool vec_ok =
      ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  if (vec_ok) {
    const int64_t nv = n >> 4;
    auto put = [&](int64_t i, uint4 v) {
      if (target == TO_ALL_MC) {
        multimem_st16(ctx.mc + staging_off + (i << 4), v);
      } else if (target == TO_ALL_LOOP) {
        for (int p = 0; p < ctx.world; ++p)
          st16(ctx.peers[p] + staging_off + (i << 4), v);
      } else {
        st16(reinterpret_cast<uint4*>(dst) + i, v);
      }
    };
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    int64_t i = threadIdx.x;
    // Four loads in flight per thread before the first store.
    for (; i + 3 * THREADS < nv; i += 4 * THREADS) {
      const uint4 a = ld16(s4 + i), b = ld16(s4 + i + THREADS);
      const uint4 c = ld16(s4 + i + 2 * THREADS), d = ld16(s4 + i + 3 * THREADS);
      put(i, a);
      put(i + THREADS, b);
      put(i + 2 * THREADS, c);
      put(i + 3 * THREADS, d);
    }
    for (; i < nv; i += THREADS) put(i, ld16(s4 + i));
    src += nv << 4;
    dst += nv << 4;
    staging_off += nv << 4;
    n -= nv << 4;
  }
  // Tail, or everything when the pointers are not 16-byte aligned.
  for (int64_t i = threadIdx.x; i < n; i += THREADS) {
    const char c = src[i];
    if (target == TO_ALL_MC || target == TO_ALL_LOOP) {
      for (int p = 0; p < ctx.world; ++p)
        reinterpret_cast<volatile char*>(ctx.peers[p] + staging_off)[i] = c;
    } else {
      reinterpret_cast<volatile char*>(dst)[i] = c;
    }
  }
}

}  // namespace exch
}  // namespace kern
}  // namespace hvd
