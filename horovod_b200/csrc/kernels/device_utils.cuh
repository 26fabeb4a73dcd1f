// Device-side building blocks shared by the collective kernels: system-scope
// flag loads/stores, the bounded cross-GPU CTA barrier, 16-byte vector
// loads/stores that bypass L1, NVLink multimem reductions/stores, and
// conversions between tensor and wire element types.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "kernels.h"

namespace hvd {
namespace kern {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// 16-byte accesses that skip L1 (data written by other GPUs must never be
// served from a stale L1 line) but may use L2.
__device__ __forceinline__ uint4 ld16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st16(void* p, uint4 v) {
  asm volatile("st.global.cg.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Streaming variants for tensor storage that is touched once.
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st16_stream(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- multimem (NVLink SHARP) ------------------------------------------------
// One instruction reads the same 16 bytes from every GPU bound to the
// multicast object and returns their sum / writes 16 bytes to all of them.
template <typename TWire> struct Multimem;

template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 "
        "{%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile(
        "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 "
        "{%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Phase timestamp for the optional kernel trace (one thread per launch).
__device__ __forceinline__ void trace_mark(const SymmCtx& ctx, int slot) {
  if (ctx.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0)
    *reinterpret_cast<volatile unsigned long long*>(ctx.trace + slot) = globaltimer_ns();
}

// ---- cross-GPU CTA barrier --------------------------------------------------
// CTA `block` of every rank meets CTA `block` of every other rank. Flags are
// indexed [source rank][block]; the value written is the epoch of this
// barrier, and waiting compares with wrap-around-safe arithmetic so that
// stale values from earlier launches never satisfy a later wait.
// All threads of the CTA must call it. Returns false if a peer did not show
// up within ctx.timeout_ns; the status record then names the peer.
__device__ __forceinline__ bool cta_barrier(const SymmCtx& ctx, uint32_t epoch,
                                            int block, int phase) {
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < ctx.world) {
    const int p = threadIdx.x;
    // The release is cumulative: it also publishes what the other threads of
    // the CTA wrote before the __syncthreads() above.
    st_release_sys(ctx.flags_peers[p] + ctx.rank * SYMM_MAX_BLOCKS + block, epoch);
    const uint32_t* f = ctx.flags_local + p * SYMM_MAX_BLOCKS + block;
    const unsigned long long t0 = globaltimer_ns();
    int spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
      if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
        ok = false;
        // Plain stores into host-mapped memory: several CTAs may report,
        // any one of them is a valid diagnosis. The code goes last.
        volatile int* st = ctx.status;
        st[1] = p;
        st[2] = phase;
        st[3] = block;
        __threadfence_system();
        if (st[0] == 0) st[0] = 1;  // never hide an earlier, more specific report
        __threadfence_system();
        break;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// Barrier for kernels that address symmetric-heap tensors by offset: every
// CTA also exchanges a token derived from the offsets (and the epoch, so a stale
// token never matches). A rank whose peers were not given the same symmetric
// tensors reports code 2 instead of reading unrelated memory as gradients.
__device__ __forceinline__ uint32_t symm_token(uint32_t epoch, int64_t a, int64_t b, int n) {
  uint32_t h = epoch * 2654435761u;
  h ^= static_cast<uint32_t>(a >> 4) + 0x9e3779b9u + (h << 6) + (h >> 2);
  h ^= static_cast<uint32_t>(a >> 36) + 0x9e3779b9u + (h << 6) + (h >> 2);
  h ^= static_cast<uint32_t>(b >> 4) + 0x9e3779b9u + (h << 6) + (h >> 2);
  h ^= static_cast<uint32_t>(n) + 0x9e3779b9u + (h << 6) + (h >> 2);
  return h;
}
__device__ __forceinline__ bool cta_barrier_token(const SymmCtx& ctx, uint32_t epoch,
                                                  int block, int phase, uint32_t token) {
  // Mailbox = flag bank 1, indexed like the flags: [source rank][block].
  constexpr int MAILBOX = SYMM_MAX_RANKS * SYMM_MAX_BLOCKS;
  if (threadIdx.x < ctx.world) {
    // The same thread stores the token and then releases the flag to that peer.
    volatile uint32_t* box =
        ctx.flags_peers[threadIdx.x] + MAILBOX + ctx.rank * SYMM_MAX_BLOCKS + block;
    *box = token;
  }
  if (!cta_barrier(ctx, epoch, block, phase)) return false;
  bool ok = true;
  if (threadIdx.x < ctx.world) {
    const uint32_t theirs =
        ld_acquire_sys(ctx.flags_local + MAILBOX + threadIdx.x * SYMM_MAX_BLOCKS + block);
    if (theirs != token) {
      ok = false;
      volatile int* st = ctx.status;
      st[1] = threadIdx.x;
      st[2] = phase;
      st[3] = block;
      __threadfence_system();
      st[0] = 2;
      __threadfence_system();
    }
  }
  return __syncthreads_and(ok) != 0;
}

// ---- element conversions ----------------------------------------------------
template <typename T> __device__ __forceinline__ float to_float(T v) {
  return static_cast<float>(v);
}
template <> __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_float(float v) {
  return static_cast<T>(v);
}
template <> __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float(float v) {
  return __float2bfloat16_rn(v);
}

// A 16-byte register image of wire elements.
template <typename TWire> struct WireVec {
  static constexpr int N = 16 / sizeof(TWire);
  union {
    uint4 raw;
    TWire e[N];
  };
};

// Accumulation type per wire type: 16-bit floats add in fp32, everything
// else in its own type.
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };

template <typename A, typename T> __device__ __forceinline__ A to_acc(T v) {
  return static_cast<A>(v);
}
template <> __device__ __forceinline__ float to_acc<float, __half>(__half v) {
  return __half2float(v);
}
template <> __device__ __forceinline__ float to_acc<float, __nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T, typename A> __device__ __forceinline__ T from_acc(A v) {
  return static_cast<T>(v);
}
template <> __device__ __forceinline__ __half from_acc<__half, float>(float v) {
  return __float2half_rn(v);
}
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) {
  return __float2bfloat16_rn(v);
}

}  // namespace kern
}  // namespace hvd
