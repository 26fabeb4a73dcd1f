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

__device__ __forceinline__ const void* ldg_ptr(const void* const* p) {
  return reinterpret_cast<const void*>(
      __ldg(reinterpret_cast<const unsigned long long*>(p)));
}
__device__ __forceinline__ const void* ldg_ptr(void* const* p) {
  return reinterpret_cast<const void*>(
      __ldg(reinterpret_cast<const unsigned long long*>(p)));
}

// First tensor whose range may contain fused element `elem`.
__device__ __forceinline__ int find_tensor(const TensorList& tl, int64_t elem) {
  int lo = 0, hi = tl.n - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (__ldg(tl.offsets + mid) <= elem) lo = mid; else hi = mid - 1;
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
  while (cur + 1 < tl.n && elem >= __ldg(tl.offsets + cur + 1)) ++cur;
  const int64_t local = elem - __ldg(tl.offsets + cur);
  const int64_t cnt = __ldg(tl.counts + cur);
  const T* src = static_cast<const T*>(ldg_ptr(tl.in + cur));
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
  while (cur + 1 < tl.n && elem >= __ldg(tl.offsets + cur + 1)) ++cur;
  const int64_t local = elem - __ldg(tl.offsets + cur);
  const int64_t cnt = __ldg(tl.counts + cur);
  T* dst = static_cast<T*>(const_cast<void*>(ldg_ptr(tl.out + cur)));
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
