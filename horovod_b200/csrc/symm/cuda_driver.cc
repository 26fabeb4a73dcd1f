#include "cuda_driver.h"

#include <cuda_runtime_api.h>

#include <mutex>

namespace hvd {

namespace {

DriverApi g_api;
bool g_ok = false;
std::string g_error;
std::once_flag g_once;

template <typename Fn>
bool Resolve(const char* name, Fn* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
    cudaGetLastError();
    g_error = std::string("driver entry point ") + name + " not available";
    return false;
  }
  *out = reinterpret_cast<Fn>(fn);
  return true;
}

void Load() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    cudaGetLastError();
    g_error = "no CUDA device";
    return;
  }
  bool ok = true;
  ok = ok && Resolve("cuMemCreate", &g_api.MemCreate);
  ok = ok && Resolve("cuMemRelease", &g_api.MemRelease);
  ok = ok && Resolve("cuMemAddressReserve", &g_api.MemAddressReserve);
  ok = ok && Resolve("cuMemAddressFree", &g_api.MemAddressFree);
  ok = ok && Resolve("cuMemMap", &g_api.MemMap);
  ok = ok && Resolve("cuMemUnmap", &g_api.MemUnmap);
  ok = ok && Resolve("cuMemSetAccess", &g_api.MemSetAccess);
  ok = ok && Resolve("cuMemExportToShareableHandle",
                     &g_api.MemExportToShareableHandle);
  ok = ok && Resolve("cuMemImportFromShareableHandle",
                     &g_api.MemImportFromShareableHandle);
  ok = ok && Resolve("cuMemGetAllocationGranularity",
                     &g_api.MemGetAllocationGranularity);
  ok = ok && Resolve("cuDeviceGet", &g_api.DeviceGet);
  ok = ok && Resolve("cuDeviceGetAttribute", &g_api.DeviceGetAttribute);
  ok = ok && Resolve("cuGetErrorString", &g_api.GetErrorString);
  if (!ok) return;
  // Multicast is optional: without it the P2P kernels still work.
  bool mc = Resolve("cuMulticastCreate", &g_api.MulticastCreate) &&
            Resolve("cuMulticastAddDevice", &g_api.MulticastAddDevice) &&
            Resolve("cuMulticastBindMem", &g_api.MulticastBindMem) &&
            Resolve("cuMulticastUnbind", &g_api.MulticastUnbind) &&
            Resolve("cuMulticastGetGranularity", &g_api.MulticastGetGranularity);
  if (!mc) {
    g_api.MulticastCreate = nullptr;
    g_error.clear();
  }
  g_ok = true;
}

}  // namespace

const DriverApi* GetDriverApi(std::string* error) {
  std::call_once(g_once, Load);
  if (!g_ok) {
    if (error) *error = g_error;
    return nullptr;
  }
  return &g_api;
}

std::string DriverErrorString(const DriverApi* api, CUresult r) {
  const char* s = nullptr;
  if (api && api->GetErrorString && api->GetErrorString(r, &s) == CUDA_SUCCESS && s)
    return std::string(s) + " (" + std::to_string(static_cast<int>(r)) + ")";
  return "CUDA driver error " + std::to_string(static_cast<int>(r));
}

}  // namespace hvd
