#include "topology.h"

#include <dlfcn.h>

#include <sstream>

#include <cuda_runtime_api.h>

#include "cuda_driver.h"

namespace hvd {

namespace {

// Minimal NVML surface, resolved at run time. Only read-only queries.
struct Nvml {
  void* lib = nullptr;
  int (*Init)() = nullptr;
  int (*Shutdown)() = nullptr;
  int (*GetHandleByPciBusId)(const char*, void**) = nullptr;
  int (*GetNvLinkState)(void*, unsigned, unsigned*) = nullptr;
  bool Load() {
    lib = dlopen("libnvidia-ml.so.1", RTLD_NOW);
    if (lib == nullptr) return false;
    Init = reinterpret_cast<int (*)()>(dlsym(lib, "nvmlInit_v2"));
    Shutdown = reinterpret_cast<int (*)()>(dlsym(lib, "nvmlShutdown"));
    GetHandleByPciBusId = reinterpret_cast<int (*)(const char*, void**)>(
        dlsym(lib, "nvmlDeviceGetHandleByPciBusId_v2"));
    GetNvLinkState = reinterpret_cast<int (*)(void*, unsigned, unsigned*)>(
        dlsym(lib, "nvmlDeviceGetNvLinkState"));
    return Init && Shutdown && GetHandleByPciBusId && GetNvLinkState;
  }
};

}  // namespace

GpuTopology DiscoverTopology() {
  GpuTopology t;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return t;
  }
  t.device_count = n;
  const DriverApi* api = GetDriverApi(nullptr);
  Nvml nvml;
  bool have_nvml = n > 0 && nvml.Load() && nvml.Init() == 0;
  for (int i = 0; i < n; ++i) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, i) == cudaSuccess) {
      t.names.push_back(prop.name);
      t.sm_counts.push_back(prop.multiProcessorCount);
      t.memory_bytes.push_back(static_cast<long long>(prop.totalGlobalMem));
    } else {
      cudaGetLastError();
      t.names.push_back("?");
      t.sm_counts.push_back(0);
      t.memory_bytes.push_back(0);
    }
    int mc = -1;
    if (api != nullptr) {
      CUdevice dev;
      int v = 0;
      if (api->DeviceGet(&dev, i) == CUDA_SUCCESS &&
          api->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) ==
              CUDA_SUCCESS)
        mc = v;
    }
    t.multicast_supported.push_back(mc);
    int links = -1;
    if (have_nvml) {
      char bus[32] = {};
      void* handle = nullptr;
      if (cudaDeviceGetPCIBusId(bus, sizeof(bus), i) == cudaSuccess &&
          nvml.GetHandleByPciBusId(bus, &handle) == 0) {
        links = 0;
        for (unsigned l = 0; l < 18; ++l) {
          unsigned active = 0;
          if (nvml.GetNvLinkState(handle, l, &active) == 0 && active) ++links;
        }
      }
    }
    t.nvlink_active_links.push_back(links);
  }
  if (have_nvml) nvml.Shutdown();
  t.peer_access.assign(n, std::vector<int>(n, 0));
  t.native_atomics.assign(n, std::vector<int>(n, 0));
  t.performance_rank.assign(n, std::vector<int>(n, 0));
  t.all_pairs_peer = n > 0;
  for (int i = 0; i < n; ++i) {
    for (int j = 0; j < n; ++j) {
      if (i == j) {
        t.peer_access[i][j] = 1;
        continue;
      }
      int v = 0;
      if (cudaDeviceCanAccessPeer(&v, i, j) != cudaSuccess) cudaGetLastError();
      t.peer_access[i][j] = v;
      if (!v) t.all_pairs_peer = false;
      int a = 0, r = 0;
      if (cudaDeviceGetP2PAttribute(&a, cudaDevP2PAttrNativeAtomicSupported, i, j) !=
          cudaSuccess)
        cudaGetLastError();
      if (cudaDeviceGetP2PAttribute(&r, cudaDevP2PAttrPerformanceRank, i, j) != cudaSuccess)
        cudaGetLastError();
      t.native_atomics[i][j] = a;
      t.performance_rank[i][j] = r;
    }
  }
  return t;
}

std::string GpuTopology::Summary() const {
  std::ostringstream s;
  s << device_count << " GPU(s)";
  if (device_count > 0) {
    s << " [" << names[0] << ", " << sm_counts[0] << " SMs, "
      << (memory_bytes[0] >> 30) << " GiB]";
    s << ", all-pairs peer access: " << (all_pairs_peer ? "yes" : "no");
    s << ", NVLink multicast: "
      << (multicast_supported[0] > 0 ? "yes" : multicast_supported[0] == 0 ? "no" : "unknown");
    if (nvlink_active_links[0] >= 0)
      s << ", active NVLink links on GPU 0: " << nvlink_active_links[0];
  }
  return s.str();
}

}  // namespace hvd
