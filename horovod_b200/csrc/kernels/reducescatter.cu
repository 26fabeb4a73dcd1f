// Fused reduce-scatter over NVLink: the input tensor is packed (prescaled)
// into the local staging buffer shard by shard, each shard starting on a
// 256-byte boundary; after one cross-GPU barrier rank r sums shard r from
// every peer (peer loads, or one multimem.ld_reduce per 16 bytes) and writes
// the postscaled result directly into its output tensor. Shards may be
// ragged (the first dim0 % size ranks own one extra row).
//
// Replaces ncclReduceScatter + ncclReduce for the remainder
// (horovod/common/ops/nccl_operations.cc:342,356) and backs the public
// reducescatter op.
#include "tensor_walk.cuh"

namespace hvd {
namespace kern {

namespace {

constexpr int THREADS = 512;

// Sum of 16-byte vector `idx` (relative to the arena base) over all ranks.
template <typename T, bool NVLS, int WORLD>
__device__ __forceinline__ uint4 fetch_sum(const SymmCtx& ctx, int64_t idx) {
  if constexpr (NVLS) {
    return Multimem<T>::ld_reduce(reinterpret_cast<const uint4*>(ctx.mc) + idx);
  } else {
    uint4 x[WORLD];
#pragma unroll
    for (int p = 0; p < WORLD; ++p)
      x[p] = ld16(reinterpret_cast<const uint4*>(ctx.peers[p]) + idx);
    VecAcc<T> acc;
    acc.zero();
#pragma unroll
    for (int p = 0; p < WORLD; ++p) acc.add(x[p]);
    return acc.pack();
  }
}

// Reduces vectors [lo, hi) of this rank's shard (n elements, first vector at
// arena vector index `base`) and writes them, postscaled, to `out`.
template <typename T, bool NVLS, int WORLD, int UNROLL>
__device__ __forceinline__ void reduce_shard(const SymmCtx& ctx, int64_t base, int64_t lo,
                                             int64_t hi, int64_t n, T* out,
                                             typename ScaleT<T>::type postscale, bool post) {
  constexpr int N = 16 / sizeof(T);
  auto scaled = [&](uint4 raw) {
    if (!post) return raw;
    WireVec<T> w;
    w.raw = raw;
#pragma unroll
    for (int i = 0; i < N; ++i) w.e[i] = scale_cast<T>(w.e[i], postscale, true);
    return w.raw;
  };
  const bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const int64_t vfull = aligned ? max(lo, min(hi, n / N)) : lo;
  uint4* o4 = reinterpret_cast<uint4*>(out);
  int64_t v = lo + threadIdx.x;
  for (; v + (UNROLL - 1) * THREADS < vfull; v += UNROLL * THREADS) {
    uint4 x[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      x[u] = fetch_sum<T, NVLS, WORLD>(ctx, base + v + u * THREADS);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) st16_stream(o4 + v + u * THREADS, scaled(x[u]));
  }
  for (; v < vfull; v += THREADS)
    st16_stream(o4 + v, scaled(fetch_sum<T, NVLS, WORLD>(ctx, base + v)));
  // Ragged last vector, or an output that is not 16-byte aligned.
  for (v = vfull + threadIdx.x; v < hi; v += THREADS) {
    WireVec<T> w;
    w.raw = scaled(fetch_sum<T, NVLS, WORLD>(ctx, base + v));
    const int64_t e0 = v * N;
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (e0 + i < n) out[e0 + i] = w.e[i];
  }
}

// sym_in_off >= 0: the input tensor lives in symmetric memory at that byte
// offset of every rank's arena with 16-byte aligned shard boundaries; nothing
// is staged and the shard is reduced straight out of the peers' tensors.
template <typename T, bool NVLS>
__global__ void __launch_bounds__(THREADS)
reducescatter_kernel(const T* in, T* out, const int64_t* shard_begin,
                     SymmCtx ctx, typename ScaleT<T>::type prescale,
                     typename ScaleT<T>::type postscale, int64_t sym_in_off) {
  using S = typename ScaleT<T>::type;
  constexpr int N = 16 / sizeof(T);
  const int world = ctx.world, rank = ctx.rank;
  const int b = blockIdx.x, G = gridDim.x;
  const bool pre = prescale != S(1), post = postscale != S(1);
  const bool staged = sym_in_off < 0;

  // Staging layout: shard r starts at vector index vbase[r].
  __shared__ int64_t sb[SYMM_MAX_RANKS + 1];
  __shared__ int64_t vbase[SYMM_MAX_RANKS + 1];
  if (threadIdx.x == 0) {
    int64_t v = 0;
    for (int r = 0; r <= world; ++r) {
      sb[r] = shard_begin[r];
      vbase[r] = v;
      if (r < world) {
        int64_t n = shard_begin[r + 1] - shard_begin[r];
        int64_t vecs = (n + N - 1) / N;
        v += (vecs + 15) & ~int64_t(15);  // 256-byte aligned shard starts
      }
    }
  }
  __syncthreads();
  uint4* stage = reinterpret_cast<uint4*>(ctx.local);

  // Phase 1: pack slice b of every shard.
  for (int r = 0; staged && r < world; ++r) {
    const int64_t n = sb[r + 1] - sb[r];
    const int64_t vecs = (n + N - 1) / N;
    const int64_t per = (vecs + G - 1) / G;
    const int64_t lo = b * per, hi = min(lo + per, vecs);
    const T* src = in + sb[r];
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    // Full, aligned vectors first (four loads in flight per thread), then
    // the ragged rest element by element.
    const int64_t vfull = aligned ? max(lo, min(hi, n / N)) : lo;
    {
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = stage + vbase[r];
      auto conv = [&](uint4 raw) {
        if (!pre) return raw;
        WireVec<T> w;
        w.raw = raw;
#pragma unroll
        for (int i = 0; i < N; ++i) w.e[i] = scale_cast<T>(w.e[i], prescale, true);
        return w.raw;
      };
      int64_t v = lo + threadIdx.x;
      for (; v + 3 * THREADS < vfull; v += 4 * THREADS) {
        const uint4 a = ld16_stream(s4 + v), b2 = ld16_stream(s4 + v + THREADS);
        const uint4 c = ld16_stream(s4 + v + 2 * THREADS), d = ld16_stream(s4 + v + 3 * THREADS);
        st16(d4 + v, conv(a));
        st16(d4 + v + THREADS, conv(b2));
        st16(d4 + v + 2 * THREADS, conv(c));
        st16(d4 + v + 3 * THREADS, conv(d));
      }
      for (; v < vfull; v += THREADS) st16(d4 + v, conv(ld16_stream(s4 + v)));
    }
    for (int64_t v = vfull + threadIdx.x; v < hi; v += THREADS) {
      WireVec<T> w;
      w.raw = make_uint4(0, 0, 0, 0);
      const int64_t e0 = v * N;
#pragma unroll
      for (int i = 0; i < N; ++i)
        if (e0 + i < n) w.e[i] = scale_cast<T>(src[e0 + i], prescale, pre);
      st16(stage + vbase[r] + v, w.raw);
    }
  }
  if (staged) {
    if (!cta_barrier(ctx, ctx.epoch + 1, b, 1)) return;
  } else {
    const uint32_t token = symm_token(ctx.epoch, sym_in_off, sb[world] << 4, world);
    if (!cta_barrier_token(ctx, ctx.epoch + 1, b, 1, token)) return;
  }

  // Phase 2: reduce slice b of my shard and write it out.
  {
    const int64_t n = sb[rank + 1] - sb[rank];
    const int64_t vecs = (n + N - 1) / N;
    const int64_t per = (vecs + G - 1) / G;
    const int64_t lo = b * per, hi = min(lo + per, vecs);
    // ctx.local/peers/mc point at the staging area (staged) or at the arena
    // base (symmetric input).
    const int64_t base = staged ? vbase[rank]
                                : (sym_in_off + sb[rank] * static_cast<int64_t>(sizeof(T))) >> 4;
    if constexpr (NVLS) {
      reduce_shard<T, true, 8, 4>(ctx, base, lo, hi, n, out, postscale, post);
    } else {
      switch (world) {
      case 1: reduce_shard<T, false, 1, 4>(ctx, base, lo, hi, n, out, postscale, post); break;
      case 2: reduce_shard<T, false, 2, 4>(ctx, base, lo, hi, n, out, postscale, post); break;
      case 3: reduce_shard<T, false, 3, 2>(ctx, base, lo, hi, n, out, postscale, post); break;
      case 4: reduce_shard<T, false, 4, 2>(ctx, base, lo, hi, n, out, postscale, post); break;
      case 5: reduce_shard<T, false, 5, 1>(ctx, base, lo, hi, n, out, postscale, post); break;
      case 6: reduce_shard<T, false, 6, 1>(ctx, base, lo, hi, n, out, postscale, post); break;
      case 7: reduce_shard<T, false, 7, 1>(ctx, base, lo, hi, n, out, postscale, post); break;
      default: reduce_shard<T, false, 8, 1>(ctx, base, lo, hi, n, out, postscale, post); break;
      }
    }
  }
  // Peers may still be reading this rank's data: neither the staging buffer
  // nor a symmetric input may change before everybody is through.
  cta_barrier(ctx, ctx.epoch + 2, b, 2);
}

template <typename T>
cudaError_t LaunchTyped(const void* in, void* out, const int64_t* shard_begin,
                        double prescale, double postscale, bool nvls,
                        int num_ctas, const SymmCtx& ctx, cudaStream_t stream,
                        int64_t sym_in_off) {
  using S = typename ScaleT<T>::type;
  constexpr bool can_nvls = std::is_same<T, float>::value ||
                            std::is_same<T, __half>::value ||
                            std::is_same<T, __nv_bfloat16>::value;
  if constexpr (can_nvls) {
    if (nvls && ctx.mc != nullptr) {
      reducescatter_kernel<T, true><<<num_ctas, THREADS, 0, stream>>>(
          static_cast<const T*>(in), static_cast<T*>(out), shard_begin, ctx,
          static_cast<S>(prescale), static_cast<S>(postscale), sym_in_off);
      return cudaGetLastError();
    }
  }
  reducescatter_kernel<T, false><<<num_ctas, THREADS, 0, stream>>>(
      static_cast<const T*>(in), static_cast<T*>(out), shard_begin, ctx,
      static_cast<S>(prescale), static_cast<S>(postscale), sym_in_off);
  return cudaGetLastError();
}

}  // namespace

cudaError_t LaunchFusedReducescatter(const void* in, void* out, int64_t count,
                                     const int64_t* shard_begin_dev,
                                     DataType dtype, double prescale,
                                     double postscale, bool use_nvls,
                                     int num_ctas, const SymmCtx& ctx,
                                     cudaStream_t stream, int64_t sym_in_off) {
  (void)count;
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  CountKernelLaunches(1);
#define HVD_RS(T)                                                             \
  return LaunchTyped<T>(in, out, shard_begin_dev, prescale, postscale,        \
                        use_nvls, num_ctas, ctx, stream, sym_in_off)
  switch (dtype) {
  case DataType::FLOAT32: HVD_RS(float);
  case DataType::FLOAT16: HVD_RS(__half);
  case DataType::BFLOAT16: HVD_RS(__nv_bfloat16);
  case DataType::FLOAT64: HVD_RS(double);
  case DataType::INT32: HVD_RS(int32_t);
  case DataType::INT64: HVD_RS(int64_t);
  case DataType::UINT8: HVD_RS(uint8_t);
  case DataType::INT8: HVD_RS(int8_t);
  default: return cudaErrorInvalidValue;
  }
#undef HVD_RS
}

}  // namespace kern
}  // namespace hvd

// ---------------------------------------------------------------------------
// Entry point that allocates nothing (declared in no_alloc.h).

#include "no_alloc.h"

#include <cstdio>
#include <mutex>

namespace hvd {
namespace kern {
namespace {

// Layout of the static scratch: bookkeeping first, staging data after it.
constexpr size_t NA_SHARDS_OFF = 0;       // int64[2]: shard bounds {0, count}
constexpr size_t NA_STATUS_OFF = 256;     // int[4]: timeout record (unused by a group of one)
constexpr size_t NA_FLAGS_OFF = 4096;     // uint32[SYMM_MAX_RANKS * SYMM_MAX_BLOCKS]
constexpr size_t NA_DATA_OFF = 32768;     // staging for the prescaled input
constexpr size_t NA_TOTAL = NA_DATA_OFF + HVD_B200_NOALLOC_MAX_BYTES;
static_assert(NA_FLAGS_OFF + SYMM_MAX_RANKS * SYMM_MAX_BLOCKS * 4 <= NA_DATA_OFF,
              "flag words must fit before the staging area");

// In host code this name is only a handle for the runtime's symbol table,
// never a device address: host code must go through cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NA_TOTAL];

constexpr int NA_MAX_DEVICES = 64;
std::mutex g_na_mu;
unsigned char* g_na_base[NA_MAX_DEVICES] = {};

// Resets what this call relies on: shard bounds for a group of one and the
// barrier flag words (the previous call left its epoch values there).
__global__ void noalloc_prepare_kernel(unsigned char* base, long long count) {
  int64_t* sb = reinterpret_cast<int64_t*>(base + NA_SHARDS_OFF);
  uint32_t* flags = reinterpret_cast<uint32_t*>(base + NA_FLAGS_OFF);
  int* status = reinterpret_cast<int*>(base + NA_STATUS_OFF);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    sb[0] = 0;
    sb[1] = count;
    status[0] = status[1] = status[2] = status[3] = 0;
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x;
       i < SYMM_MAX_RANKS * SYMM_MAX_BLOCKS; i += gridDim.x * blockDim.x)
    flags[i] = 0;
}

int Fail(int code, char* err, unsigned long err_len, const char* what,
         const char* detail = "") {
  if (err != nullptr && err_len > 0)
    std::snprintf(err, err_len, "hvd_b200_reducescatter1_noalloc: %s%s", what, detail);
  return code;
}

}  // namespace
}  // namespace kern
}  // namespace hvd

extern "C" __attribute__((visibility("default"))) int
hvd_b200_reducescatter1_noalloc(const void* in, void* out, long long count,
                                int dtype, double prescale, double postscale,
                                void* stream_v, char* err, unsigned long err_len) {
  using namespace hvd;
  using namespace hvd::kern;
  // Validate the id before it is narrowed to the one-byte enum.
  if (dtype < 0 || dtype > 255) return Fail(2, err, err_len, "unsupported dtype id");
  DataType dt = static_cast<DataType>(dtype);
  switch (dt) {
  case DataType::UINT8: case DataType::INT8: case DataType::INT32:
  case DataType::INT64: case DataType::FLOAT16: case DataType::FLOAT32:
  case DataType::FLOAT64: case DataType::BFLOAT16:
    break;
  default:
    return Fail(2, err, err_len, "unsupported dtype id");
  }
  if (count < 0) return Fail(2, err, err_len, "negative element count");
  if (count == 0) return 0;
  if (in == nullptr || out == nullptr)
    return Fail(2, err, err_len, "null input or output pointer");
  // Compare element counts, not a byte product that could wrap around.
  const unsigned long long elem_size = DataTypeSize(dt);
  if (static_cast<unsigned long long>(count) > HVD_B200_NOALLOC_MAX_BYTES / elem_size) {
    char detail[128];
    std::snprintf(detail, sizeof(detail),
                  " (%lld elements of %llu bytes requested, limit %u bytes)", count,
                  elem_size, static_cast<unsigned>(HVD_B200_NOALLOC_MAX_BYTES));
    return Fail(1, err, err_len, "input larger than the built-in scratch", detail);
  }
  const unsigned long long bytes = static_cast<unsigned long long>(count) * elem_size;

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return Fail(3, err, err_len, "cudaGetDevice failed: ", cudaGetErrorString(e));
  if (device < 0 || device >= NA_MAX_DEVICES)
    return Fail(3, err, err_len, "device ordinal out of range");
  unsigned char* base = nullptr;
  {
    // Once per device, with that device current: resolve the device address
    // of the static array.
    std::lock_guard<std::mutex> lock(g_na_mu);
    if (g_na_base[device] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess)
        return Fail(3, err, err_len, "cudaGetSymbolAddress failed: ",
                    cudaGetErrorString(e));
      g_na_base[device] = static_cast<unsigned char*>(p);
    }
    base = g_na_base[device];
  }

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  noalloc_prepare_kernel<<<8, 512, 0, stream>>>(base, count);
  e = cudaGetLastError();
  if (e != cudaSuccess)
    return Fail(3, err, err_len, "launch of the prepare kernel failed: ",
                cudaGetErrorString(e));

  SymmCtx ctx;
  std::memset(&ctx, 0, sizeof(ctx));
  ctx.rank = 0;
  ctx.world = 1;
  ctx.local = reinterpret_cast<char*>(base + NA_DATA_OFF);
  ctx.peers[0] = ctx.local;
  ctx.mc = nullptr;
  ctx.flags_local = reinterpret_cast<uint32_t*>(base + NA_FLAGS_OFF);
  ctx.flags_peers[0] = ctx.flags_local;
  ctx.epoch = 0;
  ctx.timeout_ns = 1000000000ull;  // a group of one never waits for anybody
  ctx.status = reinterpret_cast<int*>(base + NA_STATUS_OFF);
  const int ctas = bytes <= (64u << 10) ? 4 : 16;
  e = LaunchFusedReducescatter(
      in, out, count, reinterpret_cast<const int64_t*>(base + NA_SHARDS_OFF), dt,
      prescale, postscale, /*use_nvls=*/false, ctas, ctx, stream);
  if (e != cudaSuccess)
    return Fail(3, err, err_len, "launch of the reduce-scatter kernel failed: ",
                cudaGetErrorString(e));
  return 0;
}
