// NCCL path, part two: broadcast, allgather, alltoall, reducescatter.
#include <dlfcn.h>

#include <algorithm>
#include <cstring>

#include "../common/logging.h"
#include "../common/process_set.h"
#include "gpu_internal.h"
#include "nccl_api.h"
#include "nccl_ops.h"
#include "host_trace.h"

namespace hvd {

#define HVD_NCCL(call)                                                        \
  do {                                                                        \
    ncclResult_t r_ = (call);                                                 \
    if (r_ != ncclSuccess)                                                    \
      throw std::runtime_error(std::string(#call) + " failed: " +             \
                               api_->GetErrorString(r_));                     \
  } while (0)

Status NcclOps::Broadcast(std::vector<TensorTableEntry>& entries, void* comm_v) {
  ncclComm_t comm = static_cast<ncclComm_t>(comm_v);
  cudaStream_t stream = gpu_.stream();
  Timeline& tl = gpu_.state().timeline;
  for (auto& e : entries) {
    gpu_.ActStart(e.name, HVD_ACT_NCCL_BCAST);
    host_trace::Mark("before call");
    HVD_NCCL(api_->Broadcast(e.input, e.output, static_cast<size_t>(e.size_bytes()),
                             ncclChar, e.root_rank, comm, stream));
    host_trace::Mark("nccl call");
    gpu_.ActEnd(e.name);
  }
  return gpu_.Complete(entries);
}

Status NcclOps::Allgather(std::vector<TensorTableEntry>& entries,
                          const Response& response, ProcessSet& ps,
                          void* comm_v) {
  ncclComm_t comm = static_cast<ncclComm_t>(comm_v);
  cudaStream_t stream = gpu_.stream();
  Timeline& tl = gpu_.state().timeline;
  const int n = ps.comm.size(), me = ps.comm.rank();
  for (size_t i = 0; i < entries.size(); ++i) {
    TensorTableEntry& e = entries[i];
    int64_t slice = static_cast<int64_t>(DataTypeSize(e.dtype));
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    int64_t rows = 0;
    bool equal = true;
    for (int r = 0; r < n; ++r) {
      rows += response.tensor_sizes[i * n + r];
      equal = equal && response.tensor_sizes[i * n + r] == response.tensor_sizes[i * n];
    }
    std::vector<int64_t> dims = e.shape.to_vector();
    dims[0] = rows;
    void* out = nullptr;
    Status st = e.context->AllocateOutput(TensorShape(dims), stream, &out);
    if (!st.ok()) return st;
    e.output = out;
    gpu_.ActStart(e.name, HVD_ACT_NCCL_ALLGATHER);
    if (equal) {
      host_trace::Mark("before call");
      HVD_NCCL(api_->AllGather(e.input, out,
                               static_cast<size_t>(response.tensor_sizes[i * n] * slice),
                               ncclChar, comm, stream));
      host_trace::Mark("nccl call");
    } else {
      // Unequal contributions: one broadcast per rank, grouped.
      HVD_NCCL(api_->GroupStart());
      int64_t disp = 0;
      for (int r = 0; r < n; ++r) {
        int64_t bytes = response.tensor_sizes[i * n + r] * slice;
        char* dst = static_cast<char*>(out) + disp;
        const void* src = r == me ? e.input : dst;
        if (bytes > 0)
          HVD_NCCL(api_->Broadcast(src, dst, static_cast<size_t>(bytes), ncclChar,
                                   r, comm, stream));
        disp += bytes;
      }
      HVD_NCCL(api_->GroupEnd());
    }
    gpu_.ActEnd(e.name);
  }
  return gpu_.Complete(entries);
}

Status NcclOps::Alltoall(std::vector<TensorTableEntry>& entries, const Response& response,
                         ProcessSet& ps, void* comm_v) {
  ncclComm_t comm = static_cast<ncclComm_t>(comm_v);
  cudaStream_t stream = gpu_.stream();
  Timeline& tl = gpu_.state().timeline;
  const int n = ps.comm.size();
  for (auto& e : entries) {
    int64_t slice = static_cast<int64_t>(DataTypeSize(e.dtype));
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    std::vector<int32_t> recv(n);
    if (!AlltoallEvenRows(response, n, &recv)) {
      std::vector<int64_t> four(n, 4);
      ps.comm.Alltoallv(e.splits.data(), four, recv.data(), four);
    }
    int64_t rows = 0;
    for (int r = 0; r < n; ++r) rows += recv[r];
    std::vector<int64_t> dims = e.shape.to_vector();
    dims[0] = rows;
    void* out = nullptr;
    Status st = e.context->AllocateOutput(TensorShape(dims), stream, &out);
    if (!st.ok()) return st;
    e.output = out;
    e.context->SetReceivedSplits(recv);
    gpu_.ActStart(e.name, HVD_ACT_NCCL_ALLTOALL);
    HVD_NCCL(api_->GroupStart());
    int64_t soff = 0, roff = 0;
    for (int p = 0; p < n; ++p) {
      int64_t sb = e.splits[p] * slice, rb = recv[p] * slice;
      if (sb > 0)
        HVD_NCCL(api_->Send(static_cast<const char*>(e.input) + soff,
                            static_cast<size_t>(sb), ncclChar, p, comm, stream));
      if (rb > 0)
        HVD_NCCL(api_->Recv(static_cast<char*>(out) + roff, static_cast<size_t>(rb),
                            ncclChar, p, comm, stream));
      soff += sb;
      roff += rb;
    }
    HVD_NCCL(api_->GroupEnd());
    gpu_.ActEnd(e.name);
  }
  return gpu_.Complete(entries);
}

Status NcclOps::Reducescatter(std::vector<TensorTableEntry>& entries,
                              ProcessSet& ps, void* comm_v) {
  ncclComm_t comm = static_cast<ncclComm_t>(comm_v);
  cudaStream_t stream = gpu_.stream();
  Timeline& tl = gpu_.state().timeline;
  const int n = ps.comm.size(), me = ps.comm.rank();
  for (auto& e : entries) {
    ncclDataType_t nt;
    switch (e.dtype) {
    case DataType::UINT8: nt = ncclUint8; break;
    case DataType::INT8: nt = ncclInt8; break;
    case DataType::INT32: nt = ncclInt32; break;
    case DataType::INT64: nt = ncclInt64; break;
    case DataType::FLOAT16: nt = ncclFloat16; break;
    case DataType::FLOAT32: nt = ncclFloat32; break;
    case DataType::FLOAT64: nt = ncclFloat64; break;
    case DataType::BFLOAT16: nt = ncclBfloat16; break;
    default:
      return Status::InvalidArgument(std::string("NCCL cannot reduce dtype ") +
                                     DataTypeName(e.dtype));
    }
    ncclRedOp_t op = e.reduce_op == ReduceOp::MIN ? ncclMin
                     : e.reduce_op == ReduceOp::MAX ? ncclMax
                     : e.reduce_op == ReduceOp::PRODUCT ? ncclProd : ncclSum;
    const int64_t es = static_cast<int64_t>(DataTypeSize(e.dtype));
    int64_t rows = e.shape.dim_size(0), slice = 1;
    for (int d = 1; d < e.shape.dims(); ++d) slice *= e.shape.dim_size(d);
    const int64_t base = rows / n, extra = rows % n;
    const int64_t my_rows = base + (me < extra ? 1 : 0);
    const int64_t my_start = me * base + std::min<int64_t>(me, extra);
    std::vector<int64_t> dims = e.shape.to_vector();
    dims[0] = my_rows;
    void* out = nullptr;
    Status st = e.context->AllocateOutput(TensorShape(dims), stream, &out);
    if (!st.ok()) return st;
    e.output = out;
    const int64_t total = e.num_elements();
    const void* src = e.input;
    void* tmp = nullptr;
    if (e.prescale != 1.0 || extra != 0) tmp = Fusion(static_cast<size_t>(total * es));
    if (e.prescale != 1.0) {
      kern::LaunchScaleBuffer(e.input, tmp, total, e.dtype, e.prescale, stream);
      src = tmp;
    }
    gpu_.ActStart(e.name, HVD_ACT_NCCL_REDUCESCATTER);
    if (extra == 0) {
      HVD_NCCL(api_->ReduceScatter(src, out, static_cast<size_t>(base * slice), nt,
                                   op, comm, stream));
    } else {
      // Ragged shards: reduce everything, keep this rank's rows.
      HVD_NCCL(api_->AllReduce(src, tmp, static_cast<size_t>(total), nt, op, comm, stream));
      HVD_CUDA(cudaMemcpyAsync(out, static_cast<char*>(tmp) + my_start * slice * es,
                               static_cast<size_t>(my_rows * slice * es),
                               cudaMemcpyDeviceToDevice, stream));
    }
    gpu_.ActEnd(e.name);
    if (e.postscale != 1.0)
      kern::LaunchScaleBuffer(out, out, my_rows * slice, e.dtype, e.postscale, stream);
  }
  return gpu_.Complete(entries);
}

}  // namespace hvd
