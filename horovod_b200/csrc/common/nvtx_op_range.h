// NVTX ranges around every collective, from enqueue to completion, in the
// domain "HorovodOps" (visible in Nsight Systems). Disabled with
// HOROVOD_DISABLE_NVTX_RANGES=1. NVTX3 is header-only and resolves the
// profiler's injection library lazily, so nothing links against it and the
// calls are no-ops when no profiler is attached.
//
// Parity: horovod/common/nvtx_op_range.h:12-87, nvtx_op_range.cc:8-31.
#pragma once

#include <cstdint>
#include <string>

namespace hvd {

enum class NvtxOp : int {
  ALLREDUCE = 0,
  GROUPED_ALLREDUCE,
  ALLGATHER,
  BROADCAST,
  ALLTOALL,
  REDUCESCATTER,
  JOIN,
  COUNT,
};

// Opaque range id (0 = no range started).
using NvtxRangeId = uint64_t;

void NvtxSetEnabled(bool enabled);
NvtxRangeId NvtxRangeStart(NvtxOp op, const std::string& tensor_name,
                           int64_t payload_bytes);
void NvtxRangeEnd(NvtxRangeId id);

// Mirror of the timeline in NVTX: one domain for whole ops
// ("HorovodTimelineOps": tensor name + collective type from start to end of
// its execution), one for the activities inside them
// ("HorovodTimelineActivities"). Returns 0 when ranges are disabled.
// Parity: horovod/common/timeline.cc:332-425.
NvtxRangeId NvtxTimelineRangeStart(bool activity, const std::string& tensor,
                                   const std::string& name);
void NvtxTimelineRangeEnd(bool activity, NvtxRangeId id);

}  // namespace hvd
