// A single entry point for callers that are not allowed to allocate device
// memory.
//
// This function has no counterpart in the reference (uber/horovod): it exists
// for embedders of this library's kernels that run where cudaMalloc is off
// limits. Two kinds of caller are meant:
//   * a process whose device memory has been handed out in full to another
//     owner (a serving runtime that pre-plans every byte, or a framework
//     allocator that reserved the whole GPU), so a late cudaMalloc fails or
//     fragments somebody else's plan;
//   * code on a latency-critical or restricted path (inside a library
//     callback, a real-time loop, a region where implicit device
//     synchronisation is forbidden) where cudaMalloc's device-wide
//     synchronisation and unbounded latency are not acceptable.
// The ordinary entry points of this library obtain their staging memory from
// a symmetric arena created with the CUDA virtual-memory API; this one uses a
// fixed array that is part of the loaded module instead.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest input, in bytes, that the entry point accepts.
#define HVD_B200_NOALLOC_MAX_BYTES (4u << 20)

// Single-rank reduce-scatter (a group of one): out[i] = postscale *
// (prescale * in[i]) for `count` elements of type `dtype`, computed by the
// library's reduce-scatter kernel, which stages the prescaled input in
// scratch memory before reducing and writing the result. `in` and `out` are
// device pointers supplied by the caller (they may be equal); `stream` is a
// cudaStream_t (null = the default stream). `dtype` uses the library's wire
// ids: 0 uint8, 1 int8, 4 int32, 5 int64, 6 float16, 7 float32, 8 float64,
// 10 bfloat16.
//
// Memory: the scratch is a file-scope `static __device__` array of
// HVD_B200_NOALLOC_MAX_BYTES plus 32 KiB of bookkeeping. Every GPU that loads
// the library carries it until the process exits. The function calls no
// cudaMalloc, cudaFree or any allocating library routine.
//
// First call on a device: looks up the device address of the scratch array
// (cudaGetSymbolAddress, with that device current) and remembers it. Make
// that first call before starting any stream capture on the device.
//
// Sharing: all calls on a device use the same scratch, which still holds
// whatever the previous call left there; each call re-initialises the
// bookkeeping words it depends on. Two calls whose work overlaps on the GPU
// (different streams without an ordering between them) race on the scratch:
// order them.
//
// Returns 0 on success. On failure returns a non-zero code and, if `err` is
// non-null, writes a NUL-terminated explanation into err[0..err_len):
//   1  count * sizeof(dtype) exceeds HVD_B200_NOALLOC_MAX_BYTES
//   2  unsupported dtype, negative count, or null pointer with count > 0
//   3  a CUDA call failed (message names it)
int hvd_b200_reducescatter1_noalloc(const void* in, void* out, long long count,
                                    int dtype, double prescale,
                                    double postscale, void* stream, char* err,
                                    unsigned long err_len);

#ifdef __cplusplus
}
#endif
