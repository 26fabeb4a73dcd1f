// Helpers shared by the exchange kernel: how a segment is divided among the
// CTAs of a launch, and cooperative byte copies between tensor storage of any
// alignment and the 256-byte aligned exchange regions.
#pragma once

#include "device_utils.cuh"

namespace hvd {
namespace kern {
namespace exch {

constexpr int THREADS = 512;
constexpr int64_t SMALL_SEGMENT = 64 * 1024;

// Byte range of a segment that CTA b is responsible for. Small segments are
// owned by one CTA (chosen from their region offset, which both sides know);
// larger ones are split evenly on 256-byte boundaries.
__device__ __forceinline__ void my_range(int64_t region_off, int64_t bytes,
                                         int b, int G, int64_t* lo, int64_t* hi) {
  if (bytes <= SMALL_SEGMENT) {
    const int owner = static_cast<int>((region_off >> 8) % G);
    *lo = 0;
    *hi = owner == b ? bytes : 0;
    return;
  }
  int64_t slice = (bytes + G - 1) / G;
  slice = (slice + 255) & ~int64_t(255);
  *lo = min(bytes, b * slice);
  *hi = min(bytes, *lo + slice);
}

// Widest access both the address and the remaining length allow: 16, 4 or 1.
__device__ __forceinline__ int align_class(const void* p) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  return (a & 15) == 0 ? 16 : (a & 3) == 0 ? 4 : 1;
}

// 16 bytes starting at p, of which only the first `valid` may be read.
__device__ __forceinline__ uint4 load16_any(const char* p, int cls, int valid) {
  if (cls == 16 && valid >= 16) return ld16(p);
  union {
    uint4 v;
    uint32_t w[4];
    unsigned char c[16];
  } u;
  u.v = make_uint4(0, 0, 0, 0);
  if (cls >= 4) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
    int i = 0;
#pragma unroll
    for (; i < 4; ++i)
      if (4 * i + 4 <= valid) u.w[i] = __ldcg(q + i);
    for (int j = (valid & ~3); j < valid; ++j) u.c[j] = p[j];
  } else {
    for (int j = 0; j < 16; ++j)
      if (j < valid) u.c[j] = p[j];
  }
  return u.v;
}

// Writes the first `valid` bytes of v to p.
__device__ __forceinline__ void store16_any(char* p, int cls, int valid, uint4 v) {
  if (cls == 16 && valid >= 16) {
    st16(p, v);
    return;
  }
  union {
    uint4 v;
    uint32_t w[4];
    unsigned char c[16];
  } u;
  u.v = v;
  if (cls >= 4) {
    uint32_t* q = reinterpret_cast<uint32_t*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (4 * i + 4 <= valid) __stcg(q + i, u.w[i]);
    for (int j = (valid & ~3); j < valid; ++j) p[j] = u.c[j];
  } else {
    for (int j = 0; j < 16; ++j)
      if (j < valid) p[j] = u.c[j];
  }
}

// Cooperative copy of n bytes from src to up to two destinations:
//   region  16-byte aligned address inside an exchange region (null = none);
//           whole vectors are written, so up to 15 bytes of padding behind the
//           n bytes may be overwritten (regions are padded to 256 bytes);
//           written with multimem.st when `mc` is set (then it is the
//           multicast view of the region);
//   other   ordinary local memory of any alignment (null = none), exactly n
//           bytes are written.
// src may have any alignment; exactly n bytes are read, unless `src_padded`
// says that whole vectors may be read (src is itself a region).
template <int UNROLL>
__device__ __forceinline__ void copy_bytes(const char* src, bool src_padded, char* region,
                                           bool mc, char* other, int64_t n) {
  if (n <= 0) return;
  const int64_t nv = (n + 15) >> 4;  // vectors, the last one possibly partial
  const int scls = align_class(src);
  const int ocls = other != nullptr ? align_class(other) : 16;
  const int64_t full = n >> 4;  // vectors that are whole in src
  auto put = [&](int64_t i, uint4 v, int valid) {
    if (region != nullptr) {
      if (mc)
        multimem_st16(region + (i << 4), v);
      else
        st16(region + (i << 4), v);
    }
    if (other != nullptr) store16_any(other + (i << 4), ocls, valid, v);
  };
  int64_t i = threadIdx.x;
  if (scls == 16) {
    const int64_t fast = src_padded ? nv : full;
    for (; i + (UNROLL - 1) * THREADS < fast; i += UNROLL * THREADS) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ld16(src + ((i + u * THREADS) << 4));
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int64_t j = i + u * THREADS;
        put(j, v[u], j < full ? 16 : static_cast<int>(n - (j << 4)));
      }
    }
  }
  for (; i < nv; i += THREADS) {
    const int valid = i < full ? 16 : static_cast<int>(n - (i << 4));
    const uint4 v = load16_any(src + (i << 4), scls, src_padded ? 16 : valid);
    put(i, v, valid);
  }
}

}  // namespace exch
}  // namespace kern
}  // namespace hvd
