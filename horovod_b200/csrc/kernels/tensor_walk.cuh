// Moving 16-byte vectors between a list of tensors and the linear "fused"
// index space without ever materialising a separate fusion buffer pass:
// gather_vec reads one wire vector's worth of elements straight from tensor
// storage (scaling and casting on the way), scatter_vec writes one back.
// Tensor starts are 16-byte aligned in the fused space, so a vector never
// straddles two tensors; elements in the padding read as zero.
#pragma once

#include <type_traits>

#include "device_utils.cuh"

namespace hvd {
namespace kern {

// Scaling arithmetic: wide types and integers scale in double (integers
// truncate afterwards, like the host path), everything else in float.
template <typename T> struct ScaleT { using type = float; };
template <> struct ScaleT<double> { using type = double; };
template <> struct ScaleT<int32_t> { using type = double; };
template <> struct ScaleT<int64_t> { using type = double; };

template <typename W, typename T, typename S>
__device__ __forceinline__ W scale_cast(T v, S scale, bool do_scale) {
  if constexpr (std::is_integral<T>::value) {
    if (!do_scale) return static_cast<W>(v);
    return static_cast<W>(static_cast<T>(static_cast<S>(v) * scale));
  } else if constexpr (std::is_same<T, double>::value) {
    return static_cast<W>(do_scale ? v * scale : v);
  } else {
    float f = to_float(v);
    if (do_scale) f *= static_cast<float>(scale);
    return from_float<W>(f);
  }
}

// First tensor whose range may contain fused element `elem`.
__device__ __forceinline__ int find_tensor(const TensorList& tl, int64_t elem) {
  int lo = 0, hi = tl.n - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (tl.offsets[mid] <= elem) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Reads N = 16/sizeof(W) consecutive fused elements starting at `elem`
// (a multiple of N). `cur` is a cursor into the tensor list that only moves
// forward; initialise it with find_tensor().
template <typename T, typename W, typename S>
__device__ __forceinline__ uint4 gather_vec(const TensorList& tl, int& cur,
                                            int64_t elem, S scale,
                                            bool do_scale) {
  constexpr int N = 16 / sizeof(W);
  while (cur + 1 < tl.n && elem >= tl.offsets[cur + 1]) ++cur;
  const int64_t local = elem - tl.offsets[cur];
  const int64_t cnt = tl.counts[cur];
  const T* src = static_cast<const T*>(tl.in[cur]);
  WireVec<W> out;
  out.raw = make_uint4(0, 0, 0, 0);
  if (src == nullptr || local >= cnt) return out.raw;
  src += local;
  const bool full = local + N <= cnt;
  if (full && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    constexpr int LOADS = N * sizeof(T) / 16;  // 1, or 2 for fp32 -> 16-bit
    union {
      uint4 raw[LOADS];
      T e[N];
    } in;
#pragma unroll
    for (int i = 0; i < LOADS; ++i)
      in.raw[i] = ld16_stream(reinterpret_cast<const uint4*>(src) + i);
    if constexpr (std::is_same<T, W>::value) {
      if (!do_scale) return in.raw[0];
    }
#pragma unroll
    for (int i = 0; i < N; ++i) out.e[i] = scale_cast<W>(in.e[i], scale, do_scale);
  } else {
    const int n = full ? N : static_cast<int>(cnt - local);
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (i < n) out.e[i] = scale_cast<W>(src[i], scale, do_scale);
  }
  return out.raw;
}

// Writes N fused elements starting at `elem` to their tensor (elements in
// the padding are dropped).
template <typename T, typename W, typename S>
__device__ __forceinline__ void scatter_vec(const TensorList& tl, int& cur,
                                            int64_t elem, uint4 raw, S scale,
                                            bool do_scale) {
  constexpr int N = 16 / sizeof(W);
  while (cur + 1 < tl.n && elem >= tl.offsets[cur + 1]) ++cur;
  const int64_t local = elem - tl.offsets[cur];
  const int64_t cnt = tl.counts[cur];
  T* dst = static_cast<T*>(tl.out[cur]);
  if (dst == nullptr || local >= cnt) return;
  dst += local;
  WireVec<W> in;
  in.raw = raw;
  const bool full = local + N <= cnt;
  if (full && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    constexpr int STORES = N * sizeof(T) / 16;
    union {
      uint4 raw[STORES];
      T e[N];
    } out;
    if constexpr (std::is_same<T, W>::value) {
      if (!do_scale) {
        st16_stream(dst, raw);
        return;
      }
    }
#pragma unroll
    for (int i = 0; i < N; ++i) out.e[i] = scale_cast<T>(in.e[i], scale, do_scale);
#pragma unroll
    for (int i = 0; i < STORES; ++i)
      st16_stream(reinterpret_cast<uint4*>(dst) + i, out.raw[i]);
  } else {
    const int n = full ? N : static_cast<int>(cnt - local);
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (i < n) dst[i] = scale_cast<T>(in.e[i], scale, do_scale);
  }
}

// ---- range walkers ---------------------------------------------------------
// The per-vector functions above look the tensor up for every 16 bytes. The
// walkers below are what the kernels use for bulk work: the CTA goes through
// the tensors that overlap its range together, and inside one tensor runs a
// tight, four-way unrolled vector loop with no per-vector bookkeeping, so
// many loads are in flight per thread. `sink(v, raw)` receives fused vector
// index v and its 16 bytes; `source(v)` provides them.

template <typename T, typename W, typename S>
__device__ __forceinline__ uint4 convert_in(const uint4* raw, S scale, bool do_scale) {
  constexpr int N = 16 / sizeof(W);
  constexpr int LOADS = (N * sizeof(T) + 15) / 16;
  if constexpr (std::is_same<T, W>::value) {
    if (!do_scale) return raw[0];
  }
  union { uint4 r[LOADS]; T e[N]; } in;
#pragma unroll
  for (int i = 0; i < LOADS; ++i) in.r[i] = raw[i];
  WireVec<W> out;
#pragma unroll
  for (int i = 0; i < N; ++i) out.e[i] = scale_cast<W>(in.e[i], scale, do_scale);
  return out.raw;
}

template <typename T, typename W, typename S, int THREADS, int UNROLL = 4,
          typename Sink>
__device__ __forceinline__ void gather_range(const TensorList& tl, int64_t lo,
                                             int64_t hi, S scale, bool do_scale,
                                             Sink sink) {
  constexpr int N = 16 / sizeof(W);
  // Tensor elements narrower than the wire type (Adasum stages fp16 as
  // fp32) take the element-wise path; the vector path needs whole 16-byte
  // loads per wire vector.
  constexpr bool VEC = N * sizeof(T) >= 16;
  constexpr int LOADS = VEC ? N * sizeof(T) / 16 : 1;
  if (lo >= hi) return;
  for (int t = find_tensor(tl, lo * N); t < tl.n; ++t) {
    const int64_t toff = tl.offsets[t];
    if (toff >= hi * N) break;
    const int64_t tend = tl.offsets[t + 1];
    const int64_t cnt = tl.counts[t];
    const T* src = static_cast<const T*>(tl.in[t]);
    const int64_t v0 = max(lo, toff / N), v1 = min(hi, tend / N);
    // Vectors that lie entirely inside the tensor's data.
    const int64_t vfull = src ? max(v0, min(v1, (toff + cnt) / N)) : v0;
    if (VEC && src != nullptr && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      const uint4* s4 = reinterpret_cast<const uint4*>(src) - (toff / N) * LOADS;
      int64_t v = v0 + threadIdx.x;
      for (; v + (UNROLL - 1) * THREADS < vfull; v += UNROLL * THREADS) {
        uint4 raw[UNROLL][LOADS];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
          for (int i = 0; i < LOADS; ++i)
            raw[u][i] = ld16_stream(s4 + (v + u * THREADS) * LOADS + i);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          sink(v + u * THREADS, convert_in<T, W, S>(raw[u], scale, do_scale));
      }
      for (; v < vfull; v += THREADS) {
        uint4 raw[LOADS];
#pragma unroll
        for (int i = 0; i < LOADS; ++i) raw[i] = ld16_stream(s4 + v * LOADS + i);
        sink(v, convert_in<T, W, S>(raw, scale, do_scale));
      }
    } else if (src != nullptr) {
      for (int64_t v = v0 + threadIdx.x; v < vfull; v += THREADS) {
        WireVec<W> out;
        const T* p = src + (v * N - toff);
#pragma unroll
        for (int i = 0; i < N; ++i) out.e[i] = scale_cast<W>(p[i], scale, do_scale);
        sink(v, out.raw);
      }
    }
    // Ragged last vector and alignment padding (zeros).
    for (int64_t v = vfull + threadIdx.x; v < v1; v += THREADS) {
      WireVec<W> out;
      out.raw = make_uint4(0, 0, 0, 0);
      const int64_t local = v * N - toff;
      if (src != nullptr) {
#pragma unroll
        for (int i = 0; i < N; ++i)
          if (local + i < cnt) out.e[i] = scale_cast<W>(src[local + i], scale, do_scale);
      }
      sink(v, out.raw);
    }
  }
}

template <typename T, typename W, typename S>
__device__ __forceinline__ void convert_out(uint4 raw, S scale, bool do_scale, uint4* out) {
  constexpr int N = 16 / sizeof(W);
  constexpr int STORES = (N * sizeof(T) + 15) / 16;
  if constexpr (std::is_same<T, W>::value) {
    if (!do_scale) {
      out[0] = raw;
      return;
    }
  }
  WireVec<W> in;
  in.raw = raw;
  union { uint4 r[STORES]; T e[N]; } o;
#pragma unroll
  for (int i = 0; i < N; ++i) o.e[i] = scale_cast<T>(in.e[i], scale, do_scale);
#pragma unroll
  for (int i = 0; i < STORES; ++i) out[i] = o.r[i];
}

template <typename T, typename W, typename S, int THREADS, int UNROLL = 4,
          typename Source>
__device__ __forceinline__ void scatter_range(const TensorList& tl, int64_t lo,
                                              int64_t hi, S scale, bool do_scale,
                                              Source source) {
  constexpr int N = 16 / sizeof(W);
  constexpr bool VEC = N * sizeof(T) >= 16;
  constexpr int STORES = VEC ? N * sizeof(T) / 16 : 1;
  if (lo >= hi) return;
  for (int t = find_tensor(tl, lo * N); t < tl.n; ++t) {
    const int64_t toff = tl.offsets[t];
    if (toff >= hi * N) break;
    const int64_t tend = tl.offsets[t + 1];
    const int64_t cnt = tl.counts[t];
    T* dst = static_cast<T*>(tl.out[t]);
    if (dst == nullptr) continue;
    const int64_t v0 = max(lo, toff / N), v1 = min(hi, tend / N);
    const int64_t vfull = max(v0, min(v1, (toff + cnt) / N));
    if (VEC && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      uint4* d4 = reinterpret_cast<uint4*>(dst) - (toff / N) * STORES;
      int64_t v = v0 + threadIdx.x;
      for (; v + (UNROLL - 1) * THREADS < vfull; v += UNROLL * THREADS) {
        uint4 raw[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) raw[u] = source(v + u * THREADS);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          uint4 o[STORES];
          convert_out<T, W, S>(raw[u], scale, do_scale, o);
#pragma unroll
          for (int i = 0; i < STORES; ++i)
            st16_stream(d4 + (v + u * THREADS) * STORES + i, o[i]);
        }
      }
      for (; v < vfull; v += THREADS) {
        uint4 o[STORES];
        convert_out<T, W, S>(source(v), scale, do_scale, o);
#pragma unroll
        for (int i = 0; i < STORES; ++i) st16_stream(d4 + v * STORES + i, o[i]);
      }
    } else {
      for (int64_t v = v0 + threadIdx.x; v < vfull; v += THREADS) {
        WireVec<W> in;
        in.raw = source(v);
        T* p = dst + (v * N - toff);
#pragma unroll
        for (int i = 0; i < N; ++i) p[i] = scale_cast<T>(in.e[i], scale, do_scale);
      }
    }
    for (int64_t v = vfull + threadIdx.x; v < v1; v += THREADS) {
      const int64_t local = v * N - toff;
      if (local >= cnt) continue;  // pure padding
      WireVec<W> in;
      in.raw = source(v);
#pragma unroll
      for (int i = 0; i < N; ++i)
        if (local + i < cnt) dst[local + i] = scale_cast<T>(in.e[i], scale, do_scale);
    }
  }
}

// Sum of `world` wire vectors in the accumulation type of W.
template <typename W> struct VecAcc {
  using A = typename Acc<W>::type;
  static constexpr int N = 16 / sizeof(W);
  A a[N];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] = A(0);
  }
  __device__ __forceinline__ void add(uint4 raw) {
    WireVec<W> v;
    v.raw = raw;
#pragma unroll
    for (int i = 0; i < N; ++i) a[i] += to_acc<A, W>(v.e[i]);
  }
  __device__ __forceinline__ uint4 pack() const {
    WireVec<W> v;
#pragma unroll
    for (int i = 0; i < N; ++i) v.e[i] = from_acc<W, A>(a[i]);
    return v.raw;
  }
};

}  // namespace kern
}  // namespace hvd
