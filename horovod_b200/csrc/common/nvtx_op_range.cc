#include "nvtx_op_range.h"

#include <atomic>
#include <mutex>

#include <nvtx3/nvToolsExt.h>

namespace hvd {

namespace {

std::atomic<bool> g_enabled{true};
std::once_flag g_once;
nvtxDomainHandle_t g_domain = nullptr;
nvtxStringHandle_t g_names[static_cast<int>(NvtxOp::COUNT)] = {};

void Init() {
  g_domain = nvtxDomainCreateA("HorovodOps");
  static const char* names[] = {"HorovodAllreduce", "HorovodGroupedAllreduce",
                                "HorovodAllgather", "HorovodBroadcast",
                                "HorovodAlltoall", "HorovodReducescatter",
                                "HorovodJoin"};
  for (int i = 0; i < static_cast<int>(NvtxOp::COUNT); ++i)
    g_names[i] = nvtxDomainRegisterStringA(g_domain, names[i]);
}

}  // namespace

void NvtxSetEnabled(bool enabled) { g_enabled = enabled; }

NvtxRangeId NvtxRangeStart(NvtxOp op, const std::string& tensor_name,
                           int64_t payload_bytes) {
  if (!g_enabled.load(std::memory_order_relaxed)) return 0;
  std::call_once(g_once, Init);
  if (g_domain == nullptr) return 0;
  (void)tensor_name;
  nvtxEventAttributes_t attr = {};
  attr.version = NVTX_VERSION;
  attr.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
  attr.messageType = NVTX_MESSAGE_TYPE_REGISTERED;
  attr.message.registered = g_names[static_cast<int>(op)];
  attr.payloadType = NVTX_PAYLOAD_TYPE_INT64;
  attr.payload.llValue = payload_bytes;
  return nvtxDomainRangeStartEx(g_domain, &attr);
}

void NvtxRangeEnd(NvtxRangeId id) {
  if (id == 0 || g_domain == nullptr) return;
  nvtxDomainRangeEnd(g_domain, id);
}

namespace {
nvtxDomainHandle_t TimelineDomain(bool activity) {
  static nvtxDomainHandle_t ops = nvtxDomainCreateA("HorovodTimelineOps");
  static nvtxDomainHandle_t acts = nvtxDomainCreateA("HorovodTimelineActivities");
  return activity ? acts : ops;
}
}  // namespace

NvtxRangeId NvtxTimelineRangeStart(bool activity, const std::string& tensor,
                                   const std::string& name) {
  if (!g_enabled.load(std::memory_order_relaxed)) return 0;
  nvtxDomainHandle_t domain = TimelineDomain(activity);
  if (domain == nullptr) return 0;
  const std::string label = activity ? name : tensor + " " + name;
  nvtxEventAttributes_t attr = {};
  attr.version = NVTX_VERSION;
  attr.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
  attr.messageType = NVTX_MESSAGE_TYPE_ASCII;
  attr.message.ascii = label.c_str();
  return nvtxDomainRangeStartEx(domain, &attr);
}

void NvtxTimelineRangeEnd(bool activity, NvtxRangeId id) {
  if (id == 0) return;
  nvtxDomainHandle_t domain = TimelineDomain(activity);
  if (domain != nullptr) nvtxDomainRangeEnd(domain, id);
}

}  // namespace hvd
