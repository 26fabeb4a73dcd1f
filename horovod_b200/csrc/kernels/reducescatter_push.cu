// Reduce-scatter from ordinary (non-symmetric) tensors: every rank writes the
// prescaled shard that belongs to peer p straight into p's exchange region
// over NVLink (peer stores, slot [sender] of the region), chunk by chunk,
// announcing each chunk with a flag; the owner of a shard sums its own input
// with the N - 1 slots as the chunks arrive and writes the postscaled result
// into its output. The input is read once, crosses NVLink once, and nothing
// is staged locally; sending and summing overlap chunk by chunk; there is no
// barrier (a receiver waits for the chunk flags of its senders, region reuse
// is guarded by the launch credits of the exchange kernel, see
// kern::ExchangePlan).
//
// A launch handles one window [win_lo, win_hi) of element offsets inside
// every shard, so tensors larger than the region take several launches.
// Shards may be ragged (the first dim0 % size ranks own one more row).
//
// Replaces ncclReduceScatter + ncclReduce for the remainder
// (horovod/common/ops/nccl_operations.cc:342,356) for tensors outside the
// symmetric heap; reducescatter.cu covers inputs inside it.
#include "tensor_walk.cuh"

namespace hvd {
namespace kern {

namespace {

constexpr int THREADS = 512;
constexpr int CREDIT_BANK = 2 * SYMM_MAX_RANKS * SYMM_MAX_BLOCKS;

// N = 16 / sizeof(T) elements starting at element e0 of `base`, zero beyond n.
template <typename T, typename S>
__device__ __forceinline__ uint4 load_elems(const T* base, int64_t e0, int64_t n, bool aligned,
                                            S scale, bool do_scale) {
  constexpr int N = 16 / sizeof(T);
  WireVec<T> w;
  if (aligned && e0 + N <= n) {
    w.raw = ld16_stream(base + e0);
    if (do_scale) {
#pragma unroll
      for (int i = 0; i < N; ++i) w.e[i] = scale_cast<T>(w.e[i], scale, true);
    }
    return w.raw;
  }
  w.raw = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (e0 + i < n) w.e[i] = scale_cast<T>(base[e0 + i], scale, do_scale);
  return w.raw;
}

template <typename T>
__device__ __forceinline__ void store_elems(T* base, int64_t e0, int64_t n, bool aligned,
                                            uint4 raw) {
  constexpr int N = 16 / sizeof(T);
  if (aligned && e0 + N <= n) {
    st16_stream(base + e0, raw);
    return;
  }
  WireVec<T> w;
  w.raw = raw;
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (e0 + i < n) base[e0 + i] = w.e[i];
}

__device__ __forceinline__ void report(const SymmCtx& ctx, int peer, int phase, int block) {
  volatile int* st = ctx.status;
  st[1] = peer;
  st[2] = phase;
  st[3] = block;
  __threadfence_system();
  if (st[0] == 0) st[0] = 1;
  __threadfence_system();
}

template <typename T, int WORLD>
__device__ __forceinline__ void sum_chunk(const SymmCtx& ctx, const char* region, const T* mine,
                                          bool mine_aligned,
                                          T* out, bool out_aligned, int64_t n, int64_t v0,
                                          int64_t v1, int64_t slot_bytes,
                                          typename ScaleT<T>::type prescale, bool pre,
                                          typename ScaleT<T>::type postscale, bool post) {
  constexpr int N = 16 / sizeof(T);
  // Enough independent loads per thread to cover the memory latency.
  constexpr int U = WORLD <= 2 ? 4 : WORLD <= 4 ? 2 : 1;
  auto finish = [&](int64_t v, const uint4* x) {
    VecAcc<T> acc;
    acc.zero();
#pragma unroll
    for (int q = 0; q < WORLD; ++q) acc.add(x[q]);
    WireVec<T> w;
    w.raw = acc.pack();
    if (post) {
#pragma unroll
      for (int i = 0; i < N; ++i) w.e[i] = scale_cast<T>(w.e[i], postscale, true);
    }
    store_elems<T>(out, v * N, n, out_aligned, w.raw);
  };
  auto fetch = [&](int64_t v, uint4* x) {
#pragma unroll
    for (int q = 0; q < WORLD; ++q) {
      if (q == ctx.rank)
        x[q] = load_elems<T>(mine, v * N, n, mine_aligned, prescale, pre);
      else
        x[q] = ld16(region + q * slot_bytes + (v << 4));
    }
  };
  int64_t v = v0 + threadIdx.x;
  for (; v + (U - 1) * THREADS < v1; v += U * THREADS) {
    uint4 x[U][WORLD];
#pragma unroll
    for (int u = 0; u < U; ++u) fetch(v + u * THREADS, x[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) finish(v + u * THREADS, x[u]);
  }
  for (; v < v1; v += THREADS) {
    uint4 x[WORLD];
    fetch(v, x);
    finish(v, x);
  }
}

// Vectors [v0, v1) of a shard of n elements at `base`, prescaled, stored into
// a peer's slot (16 bytes per vector, same vector index).
template <typename T>
__device__ __forceinline__ void send_range(const T* base, int64_t n, int64_t v0, int64_t v1,
                                           bool aligned, char* slot,
                                           typename ScaleT<T>::type prescale, bool pre) {
  constexpr int N = 16 / sizeof(T);
  int64_t v = v0 + threadIdx.x;
  if (aligned) {
    const int64_t vfull = max(v0, min(v1, n / N));
    for (; v + 3 * THREADS < vfull; v += 4 * THREADS) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) x[u] = ld16_stream(base + (v + u * THREADS) * N);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (pre) {
          WireVec<T> w;
          w.raw = x[u];
#pragma unroll
          for (int i = 0; i < N; ++i) w.e[i] = scale_cast<T>(w.e[i], prescale, true);
          x[u] = w.raw;
        }
        st16(slot + ((v + u * THREADS) << 4), x[u]);
      }
    }
  }
  for (; v < v1; v += THREADS)
    st16(slot + (v << 4), load_elems<T>(base, v * N, n, aligned, prescale, pre));
}

template <typename T>
__device__ __forceinline__ void reducescatter_push_body(const T* in, T* out,
                                                        const RsPushArgs& args,
                                                        const SymmCtx& ctx,
                                                        typename ScaleT<T>::type prescale,
                                                        typename ScaleT<T>::type postscale) {
  using S = typename ScaleT<T>::type;
  constexpr int N = 16 / sizeof(T);
  const int world = ctx.world, rank = ctx.rank;
  const int b = blockIdx.x, G = gridDim.x;
  const bool pre = prescale != S(1), post = postscale != S(1);

  // Parameter arrays are read at compile-time offsets only.
  __shared__ int64_t sb[SYMM_MAX_RANKS + 1];
#pragma unroll
  for (int i = 0; i <= SYMM_MAX_RANKS; ++i)
    if (threadIdx.x == i) sb[i] = args.shard_begin[i];
  __syncthreads();

  if (args.credit_wait != 0) {
    bool ok = true;
    if (threadIdx.x < world) {
      const uint32_t* f = ctx.flags_local + CREDIT_BANK + threadIdx.x * SYMM_MAX_BLOCKS;
      const unsigned long long t0 = globaltimer_ns();
      int spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys(f) - args.credit_wait) < 0) {
        if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
          ok = false;
          report(ctx, threadIdx.x, 0, b);
          break;
        }
      }
    }
    if (__syncthreads_and(ok) == 0) return;
  }

  // Window of shard p: elements [sb[p] + win_lo, min(sb[p] + win_hi, sb[p+1])).
  auto window = [&](int p, const T** base, int64_t* n) {
    const int64_t len = sb[p + 1] - sb[p];
    *n = max(int64_t(0), min(len, args.win_hi) - args.win_lo);
    *base = in + sb[p] + args.win_lo;
  };
  // Slice of a window of n elements owned by this CTA, in 16-byte vectors;
  // the slice length is the same for every shard (derived from the largest).
  const int64_t Cv = args.chunk_bytes >> 4;
  const int64_t per = args.slice_vecs;  // multiple of 16 vectors
  const int64_t K = (per + Cv - 1) / Cv;
  const int64_t lo = b * per;

  for (int64_t c = 0; c <= K; ++c) {
    if (c < K) {
      // Send chunk c of every peer's shard, starting with the next rank so
      // that at any time every GPU is written by one sender.
      for (int j = 1; j < world; ++j) {
        const int p = (rank + j) % world;
        const T* base;
        int64_t n;
        window(p, &base, &n);
        const int64_t vecs = (n + N - 1) / N;
        const int64_t v0 = min(vecs, lo + c * Cv), v1 = min(vecs, min(lo + per, lo + (c + 1) * Cv));
        const bool aligned = (reinterpret_cast<uintptr_t>(base) & 15) == 0;
        char* slot = ctx.peers[p] + rank * args.slot_bytes;
        send_range<T>(base, n, v0, v1, aligned, slot, prescale, pre);
      }
      // One barrier for the chunk of all peers, then one announcing thread per
      // peer, so the release fences overlap instead of queueing up.
      __syncthreads();
      if (threadIdx.x < world && threadIdx.x != rank)
        st_release_sys(ctx.flags_peers[threadIdx.x] + rank * SYMM_MAX_BLOCKS + b,
                       ctx.epoch + static_cast<uint32_t>(c) + 1u);
    }
    if (c > 0) {
      // Sum chunk c - 1 of my shard once every sender has announced it.
      const int64_t cc = c - 1;
      const T* base;
      int64_t n;
      window(rank, &base, &n);
      const int64_t vecs = (n + N - 1) / N;
      const int64_t v0 = min(vecs, lo + cc * Cv), v1 = min(vecs, min(lo + per, lo + (cc + 1) * Cv));
      bool ok = true;
      if (v0 < v1 && threadIdx.x < world && threadIdx.x != rank) {
        const uint32_t* f = ctx.flags_local + threadIdx.x * SYMM_MAX_BLOCKS + b;
        const uint32_t want = ctx.epoch + static_cast<uint32_t>(cc) + 1u;
        const unsigned long long t0 = globaltimer_ns();
        int spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - want) < 0) {
          if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
            ok = false;
            report(ctx, threadIdx.x, 3, b);
            break;
          }
        }
      }
      if (__syncthreads_and(ok) == 0) return;
      if (v0 < v1) {
        T* o = out + args.win_lo;
        const bool ma = (reinterpret_cast<uintptr_t>(base) & 15) == 0;
        const bool oa = (reinterpret_cast<uintptr_t>(o) & 15) == 0;
        switch (world) {
#define HVD_RS_CASE(W)                                                                    \
  case W:                                                                                 \
    sum_chunk<T, W>(ctx, ctx.local, base, ma, o, oa, n, v0, v1, args.slot_bytes, prescale,  \
                    pre, postscale, post);                                                \
    break;
          HVD_RS_CASE(1) HVD_RS_CASE(2) HVD_RS_CASE(3) HVD_RS_CASE(4)
          HVD_RS_CASE(5) HVD_RS_CASE(6) HVD_RS_CASE(7)
          default:
            sum_chunk<T, 8>(ctx, ctx.local, base, ma, o, oa, n, v0, v1, args.slot_bytes,
                            prescale, pre, postscale, post);
#undef HVD_RS_CASE
        }
      }
    }
  }

  if (args.credit_post != 0) {
    // The last CTA of this rank to finish tells every peer that this launch
    // no longer reads its region (completed loads need no fence).
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0)
      s_last = atomicAdd(args.done_counter, 1ull) + 1ull == args.done_target;
    __syncthreads();
    if (s_last != 0 && threadIdx.x < world)
      st_release_sys(ctx.flags_peers[threadIdx.x] + CREDIT_BANK + rank * SYMM_MAX_BLOCKS,
                     args.credit_post);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS, 2)
reducescatter_push_kernel(const T* in, T* out, const RsPushArgs args, SymmCtx ctx,
                          typename ScaleT<T>::type prescale,
                          typename ScaleT<T>::type postscale) {
  reducescatter_push_body<T>(in, out, args, ctx, prescale, postscale);
}

// Several ranks on one GPU (tests): row y of a cooperative launch runs the
// kernel of rank y (see EmuAllreduceRank).
template <typename T>
__global__ void __launch_bounds__(THREADS, 2)
reducescatter_push_emulated_kernel(const EmuRsPushRank* ranks,
                                   typename ScaleT<T>::type prescale,
                                   typename ScaleT<T>::type postscale) {
  const EmuRsPushRank& r = ranks[blockIdx.y];
  reducescatter_push_body<T>(static_cast<const T*>(r.in), static_cast<T*>(r.out), r.args, r.ctx,
                             prescale, postscale);
}

// Several tensors in one launch. The steps of the launch are the chunks of
// all tensors in order; step g sends its chunk to every owner and announces
// it with the value epoch + g + 1, then sums the chunk of step g - 1, so the
// wait for the other senders' flags of one tensor is covered by the sending
// of the next.
struct GroupCursor {
  int t;       // tensor
  int64_t c;   // chunk inside the tensor's slice
  const char* in;
  char* out;
  int64_t base_rows, extra_rows, row_elems, slot_off, per, K;
};

__device__ __forceinline__ void cursor_load(GroupCursor& cur, const RsGroupArgs& args, int64_t Cv) {
  if (cur.t >= args.n_tensors) return;
  const RsGroupTensor* d = args.tensors + cur.t;
  cur.in = static_cast<const char*>(d->in);
  cur.out = static_cast<char*>(d->out);
  cur.base_rows = d->base_rows;
  cur.extra_rows = d->extra_rows;
  cur.row_elems = d->row_elems;
  cur.slot_off = d->slot_off;
  cur.per = d->slice_vecs;
  cur.K = (cur.per + Cv - 1) / Cv;
}

__device__ __forceinline__ void cursor_advance(GroupCursor& cur, const RsGroupArgs& args,
                                               int64_t Cv) {
  if (++cur.c < cur.K) return;
  cur.c = 0;
  ++cur.t;
  cursor_load(cur, args, Cv);
}

template <typename T>
__global__ void __launch_bounds__(THREADS, 2)
reducescatter_push_group_kernel(const RsGroupArgs args, SymmCtx ctx,
                                typename ScaleT<T>::type prescale,
                                typename ScaleT<T>::type postscale) {
  using S = typename ScaleT<T>::type;
  constexpr int N = 16 / sizeof(T);
  const int world = ctx.world, rank = ctx.rank;
  const int b = blockIdx.x;
  const bool pre = prescale != S(1), post = postscale != S(1);

  if (args.credit_wait != 0) {
    bool ok = true;
    if (threadIdx.x < world) {
      const uint32_t* f = ctx.flags_local + CREDIT_BANK + threadIdx.x * SYMM_MAX_BLOCKS;
      const unsigned long long t0 = globaltimer_ns();
      int spins = 0;
      while (static_cast<int32_t>(ld_acquire_sys(f) - args.credit_wait) < 0) {
        if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
          ok = false;
          report(ctx, threadIdx.x, 0, b);
          break;
        }
      }
    }
    if (__syncthreads_and(ok) == 0) return;
  }

  const int64_t Cv = args.chunk_bytes >> 4;
  // Elements [begin, begin + len) of the tensor belong to rank p.
  auto shard = [&](const GroupCursor& cur, int p, int64_t* begin, int64_t* len) {
    *begin = (p * cur.base_rows + min(int64_t(p), cur.extra_rows)) * cur.row_elems;
    *len = (cur.base_rows + (p < cur.extra_rows ? 1 : 0)) * cur.row_elems;
  };
  GroupCursor snd, rcv;
  snd.t = rcv.t = 0;
  snd.c = rcv.c = 0;
  cursor_load(snd, args, Cv);
  rcv = snd;

  for (uint32_t g = 0; g <= args.total_chunks; ++g) {
    if (g < args.total_chunks) {
      const int64_t lo = b * snd.per;
      for (int j = 1; j < world; ++j) {
        const int p = (rank + j) % world;
        int64_t begin, n;
        shard(snd, p, &begin, &n);
        const T* base = reinterpret_cast<const T*>(snd.in) + begin;
        const int64_t vecs = (n + N - 1) / N;
        const int64_t v0 = min(vecs, lo + snd.c * Cv);
        const int64_t v1 = min(vecs, min(lo + snd.per, lo + (snd.c + 1) * Cv));
        const bool aligned = (reinterpret_cast<uintptr_t>(base) & 15) == 0;
        char* slot = ctx.peers[p] + rank * args.slot_bytes + snd.slot_off;
        send_range<T>(base, n, v0, v1, aligned, slot, prescale, pre);
      }
      __syncthreads();
      if (threadIdx.x < world && threadIdx.x != rank)
        st_release_sys(ctx.flags_peers[threadIdx.x] + rank * SYMM_MAX_BLOCKS + b,
                       ctx.epoch + g + 1u);
      cursor_advance(snd, args, Cv);
    }
    if (g > 0) {
      const int64_t lo = b * rcv.per;
      int64_t begin, n;
      shard(rcv, rank, &begin, &n);
      const T* base = reinterpret_cast<const T*>(rcv.in) + begin;
      const int64_t vecs = (n + N - 1) / N;
      const int64_t v0 = min(vecs, lo + rcv.c * Cv);
      const int64_t v1 = min(vecs, min(lo + rcv.per, lo + (rcv.c + 1) * Cv));
      bool ok = true;
      if (v0 < v1 && threadIdx.x < world && threadIdx.x != rank) {
        const uint32_t* f = ctx.flags_local + threadIdx.x * SYMM_MAX_BLOCKS + b;
        const uint32_t want = ctx.epoch + g;
        const unsigned long long t0 = globaltimer_ns();
        int spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - want) < 0) {
          if ((++spins & 63) == 0 && globaltimer_ns() - t0 > ctx.timeout_ns) {
            ok = false;
            report(ctx, threadIdx.x, 3, b);
            break;
          }
        }
      }
      if (__syncthreads_and(ok) == 0) return;
      if (v0 < v1) {
        T* o = reinterpret_cast<T*>(rcv.out);
        const char* region = ctx.local + rcv.slot_off;
        const bool ma = (reinterpret_cast<uintptr_t>(base) & 15) == 0;
        const bool oa = (reinterpret_cast<uintptr_t>(o) & 15) == 0;
        switch (world) {
#define HVD_RS_CASE(W)                                                                    \
  case W:                                                                                 \
    sum_chunk<T, W>(ctx, region, base, ma, o, oa, n, v0, v1, args.slot_bytes, prescale,   \
                    pre, postscale, post);                                                \
    break;
          HVD_RS_CASE(1) HVD_RS_CASE(2) HVD_RS_CASE(3) HVD_RS_CASE(4)
          HVD_RS_CASE(5) HVD_RS_CASE(6) HVD_RS_CASE(7)
          default:
            sum_chunk<T, 8>(ctx, region, base, ma, o, oa, n, v0, v1, args.slot_bytes, prescale,
                            pre, postscale, post);
#undef HVD_RS_CASE
        }
      }
      cursor_advance(rcv, args, Cv);
    }
  }

  if (args.credit_post != 0) {
    __shared__ int s_last;
    __syncthreads();
    if (threadIdx.x == 0)
      s_last = atomicAdd(args.done_counter, 1ull) + 1ull == args.done_target;
    __syncthreads();
    if (s_last != 0 && threadIdx.x < world)
      st_release_sys(ctx.flags_peers[threadIdx.x] + CREDIT_BANK + rank * SYMM_MAX_BLOCKS,
                     args.credit_post);
  }
}

}  // namespace

cudaError_t LaunchReducescatterPush(const void* in, void* out, const RsPushArgs& args,
                                    DataType dtype, double prescale, double postscale,
                                    int num_ctas, const SymmCtx& ctx, cudaStream_t stream) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  if (args.chunk_bytes < 4096 || (args.chunk_bytes & 255) != 0 || (args.slice_vecs & 15) != 0 ||
      args.credit_post == 0 || args.done_counter == nullptr)
    return cudaErrorInvalidValue;
  CountKernelLaunches(1);
#define HVD_RSP(T)                                                                         \
  reducescatter_push_kernel<T><<<num_ctas, THREADS, 0, stream>>>(                          \
      static_cast<const T*>(in), static_cast<T*>(out), args, ctx,                          \
      static_cast<typename ScaleT<T>::type>(prescale),                                     \
      static_cast<typename ScaleT<T>::type>(postscale));                                   \
  return cudaGetLastError()
  switch (dtype) {
  case DataType::FLOAT32: HVD_RSP(float);
  case DataType::FLOAT16: HVD_RSP(__half);
  case DataType::BFLOAT16: HVD_RSP(__nv_bfloat16);
  case DataType::FLOAT64: HVD_RSP(double);
  case DataType::INT32: HVD_RSP(int32_t);
  case DataType::INT64: HVD_RSP(int64_t);
  case DataType::UINT8: HVD_RSP(uint8_t);
  case DataType::INT8: HVD_RSP(int8_t);
  default: return cudaErrorInvalidValue;
  }
#undef HVD_RSP
}

cudaError_t LaunchReducescatterPushEmulated(const EmuRsPushRank* ranks, int world,
                                            DataType dtype, double prescale, double postscale,
                                            int num_ctas, cudaStream_t stream) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS || world < 1 || world > SYMM_MAX_RANKS)
    return cudaErrorInvalidValue;
  CountKernelLaunches(1);
  const dim3 grid(num_ctas, world);
#define HVD_RSE(T)                                                                         \
  {                                                                                        \
    typename ScaleT<T>::type pre = static_cast<typename ScaleT<T>::type>(prescale);        \
    typename ScaleT<T>::type post = static_cast<typename ScaleT<T>::type>(postscale);      \
    void* args[] = {&ranks, &pre, &post};                                                  \
    return cudaLaunchCooperativeKernel(                                                    \
        reinterpret_cast<const void*>(&reducescatter_push_emulated_kernel<T>), grid,       \
        dim3(THREADS), args, 0, stream);                                                   \
  }
  switch (dtype) {
  case DataType::FLOAT32: HVD_RSE(float)
  case DataType::BFLOAT16: HVD_RSE(__nv_bfloat16)
  case DataType::INT32: HVD_RSE(int32_t)
  default: return cudaErrorInvalidValue;
  }
#undef HVD_RSE
}

cudaError_t LaunchReducescatterPushGroup(const RsGroupArgs& args, DataType dtype, double prescale,
                                         double postscale, int num_ctas, const SymmCtx& ctx,
                                         cudaStream_t stream) {
  if (num_ctas < 1 || num_ctas > SYMM_MAX_BLOCKS) return cudaErrorInvalidValue;
  if (args.chunk_bytes < 4096 || (args.chunk_bytes & 255) != 0 || args.n_tensors < 1 ||
      args.tensors == nullptr || args.credit_post == 0 || args.done_counter == nullptr)
    return cudaErrorInvalidValue;
  CountKernelLaunches(1);
#define HVD_RSG(T)                                                                         \
  reducescatter_push_group_kernel<T><<<num_ctas, THREADS, 0, stream>>>(                    \
      args, ctx, static_cast<typename ScaleT<T>::type>(prescale),                          \
      static_cast<typename ScaleT<T>::type>(postscale));                                   \
  return cudaGetLastError()
  switch (dtype) {
  case DataType::FLOAT32: HVD_RSG(float);
  case DataType::FLOAT16: HVD_RSG(__half);
  case DataType::BFLOAT16: HVD_RSG(__nv_bfloat16);
  case DataType::FLOAT64: HVD_RSG(double);
  case DataType::INT32: HVD_RSG(int32_t);
  case DataType::INT64: HVD_RSG(int64_t);
  case DataType::UINT8: HVD_RSG(uint8_t);
  case DataType::INT8: HVD_RSG(int8_t);
  default: return cudaErrorInvalidValue;
  }
#undef HVD_RSG
}

}  // namespace kern
}  // namespace hvd
