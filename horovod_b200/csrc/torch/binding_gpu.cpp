// Python access to device-side diagnostics and raw kernel entry points.
#include <torch/extension.h>

#include <pybind11/stl.h>

#include <cstring>

#include "../kernels/kernels.h"
#include "../ops/gpu_internal.h"
#include "../ops/gpu_ops.h"
#include "../symm/topology.h"

namespace py = pybind11;

namespace hvd {

void BindGpuDiagnostics(py::module_& m) {
  m.def("gpu_backend", &GpuBackendDescription);
  m.def("symm_empty", [](const std::vector<int64_t>& sizes, py::object dtype) {
    // A tensor inside the symmetric heap (same offset on every rank when all
    // ranks allocate the same sequence). The memory belongs to the arena: it
    // is never freed individually and dies with hvd.shutdown().
    GpuOps* ops = CurrentGpuOps();
    if (ops == nullptr)
      throw std::runtime_error("symmetric memory needs an initialised runtime with a GPU");
    at::ScalarType st = torch::python::detail::py_object_to_dtype(dtype);
    int64_t n = 1;
    for (auto d : sizes) n *= d;
    int64_t off = 0;
    void* p = ops->SymmHeapAlloc(static_cast<size_t>(std::max<int64_t>(n, 1)) *
                                     c10::elementSize(st), &off);
    if (p == nullptr)
      throw std::runtime_error(
          "symmetric heap unavailable or exhausted (backend: " + GpuBackendDescription() +
          "); raise HOROVOD_SYMM_HEAP_MB");
    auto options = at::TensorOptions().dtype(st).device(at::kCUDA, ops->device());
    return at::from_blob(p, sizes, [](void*) {}, options);
  });
  m.def("symm_heap_info", []() {
    GpuOps* ops = CurrentGpuOps();
    py::dict d;
    d["bytes"] = ops ? ops->symm_heap_bytes() : 0;
    d["used"] = ops ? ops->symm_heap_used() : 0;
    return d;
  });
  m.def("gpu_topology", []() {
    GpuTopology t = DiscoverTopology();
    py::dict d;
    d["device_count"] = t.device_count;
    d["names"] = t.names;
    d["sm_counts"] = t.sm_counts;
    d["memory_bytes"] = t.memory_bytes;
    d["multicast_supported"] = t.multicast_supported;
    d["nvlink_active_links"] = t.nvlink_active_links;
    d["peer_access"] = t.peer_access;
    d["native_atomics"] = t.native_atomics;
    d["performance_rank"] = t.performance_rank;
    d["all_pairs_peer"] = t.all_pairs_peer;
    d["summary"] = t.Summary();
    return d;
  });
  m.def("gpu_op_stats", []() {
    // (response type, payload bytes, tensors, device microseconds, host
    // microseconds from the first timing event to the last launch) of every
    // device collective since the last call; needs HOROVOD_GPU_OP_TIMING=1.
    py::list out;
    std::vector<GpuOps::OpTiming> t;
    {
      py::gil_scoped_release release;
      t = DrainAllGpuTimings();
    }
    for (auto& x : t) out.append(py::make_tuple(x.type, x.bytes, x.tensors, x.device_us, x.host_us));
    return out;
  });
  m.def("gpu_response_paths", []() {
    unsigned long long symm = 0, nccl = 0;
    GpuResponsePathCounts(&symm, &nccl);
    py::dict d;
    d["symm"] = symm;
    d["nccl"] = nccl;
    return d;
  }, "Device responses executed so far per data path: symmetric-memory kernels, NCCL.");
  m.def("bounded_wait_probe", [](int device, int timeout_ms) {
    // Runs the cross-GPU barrier kernel as rank 0 of a group of two whose
    // second member does not exist: nothing ever sets that member's flag, so
    // the wait must give up after timeout_ms and describe what it waited for
    // in the status record, leaving the context usable. This is how a dead
    // peer looks to a kernel. Returns (code, peer, phase, block, elapsed_ms).
    cudaSetDevice(device);
    const size_t flag_words = static_cast<size_t>(SYMM_FLAG_BANKS) * SYMM_MAX_RANKS * SYMM_MAX_BLOCKS;
    uint32_t* flags = nullptr;
    kern::KernelStatus* status_host = nullptr;
    int* status_dev = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&flags), flag_words * sizeof(uint32_t)) != cudaSuccess)
      throw std::runtime_error("bounded_wait_probe: cudaMalloc failed");
    cudaMemset(flags, 0, flag_words * sizeof(uint32_t));
    cudaHostAlloc(reinterpret_cast<void**>(&status_host), sizeof(kern::KernelStatus),
                  cudaHostAllocMapped);
    std::memset(status_host, 0, sizeof(kern::KernelStatus));
    cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev), status_host, 0);
    kern::SymmCtx ctx;
    std::memset(&ctx, 0, sizeof(ctx));
    ctx.rank = 0;
    ctx.world = 2;
    ctx.flags_local = flags;
    ctx.flags_peers[0] = flags;
    // The absent member's flag array: a second region of the same buffer that
    // nobody reads, so this rank's own signal does not satisfy its own wait.
    ctx.flags_peers[1] = flags + 2 * SYMM_MAX_RANKS * SYMM_MAX_BLOCKS;
    ctx.epoch = 0;
    ctx.timeout_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
    ctx.status = status_dev;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, 0);
    cudaError_t err = kern::LaunchBarrierOnly(1, 0, ctx, 0);
    cudaEventRecord(e1, 0);
    cudaError_t sync = cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    auto out = py::make_tuple(status_host->code, status_host->peer, status_host->phase,
                              status_host->block, ms, static_cast<int>(err),
                              static_cast<int>(sync));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFreeHost(status_host);
    cudaFree(flags);
    return out;
  });
  m.def("kernel_trace", []() {
    // %globaltimer (ns) at the phase boundaries of the last traced allreduce
    // kernel: 0 start, 1 packed, 2 first barrier passed, 3 reduced,
    // 4 second barrier passed, 5 unpacked. Needs HOROVOD_KERNEL_TRACE=1.
    GpuOps* ops = CurrentGpuOps();
    std::vector<unsigned long long> out;
    if (ops != nullptr && ops->kernel_trace() != nullptr)
      out.assign(ops->kernel_trace(), ops->kernel_trace() + kern::KERNEL_TRACE_SLOTS);
    return out;
  });
  m.def("kernel_launch_count", &kern::KernelLaunchCount,
        "Kernels of this library launched so far in this process.");
}

}  // namespace hvd
