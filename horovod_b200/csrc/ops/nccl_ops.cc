#include "nccl_ops.h"

#include <dlfcn.h>

#include <algorithm>
#include <cstring>

#include "../common/logging.h"
#include "../common/process_set.h"
#include "gpu_internal.h"
#include "nccl_api.h"
#include "host_trace.h"

namespace hvd {

namespace {

const NcclApi* LoadNccl(std::string* error) {
  static NcclApi api;
  static bool tried = false, ok = false;
  static std::string err;
  if (!tried) {
    tried = true;
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (lib == nullptr) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (lib == nullptr) {
      err = std::string("cannot load libnccl.so.2: ") + dlerror();
    } else {
      bool all = true;
      auto sym = [&](const char* name) {
        void* p = dlsym(lib, name);
        if (p == nullptr) {
          all = false;
          err = std::string("libnccl lacks ") + name;
        }
        return p;
      };
#define HVD_NCCL_SYM(field, name) \
  api.field = reinterpret_cast<decltype(api.field)>(sym(name))
      HVD_NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
      HVD_NCCL_SYM(CommInitRank, "ncclCommInitRank");
      HVD_NCCL_SYM(CommDestroy, "ncclCommDestroy");
      HVD_NCCL_SYM(CommAbort, "ncclCommAbort");
      HVD_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
      HVD_NCCL_SYM(GetErrorString, "ncclGetErrorString");
      HVD_NCCL_SYM(AllReduce, "ncclAllReduce");
      HVD_NCCL_SYM(Broadcast, "ncclBroadcast");
      HVD_NCCL_SYM(AllGather, "ncclAllGather");
      HVD_NCCL_SYM(ReduceScatter, "ncclReduceScatter");
      HVD_NCCL_SYM(Send, "ncclSend");
      HVD_NCCL_SYM(Recv, "ncclRecv");
      HVD_NCCL_SYM(GroupStart, "ncclGroupStart");
      HVD_NCCL_SYM(GroupEnd, "ncclGroupEnd");
#undef HVD_NCCL_SYM
      ok = all;
    }
  }
  if (!ok && error) *error = err;
  return ok ? &api : nullptr;
}

#define HVD_NCCL(call)                                                        \
  do {                                                                        \
    ncclResult_t r_ = (call);                                                 \
    if (r_ != ncclSuccess)                                                    \
      throw std::runtime_error(std::string(#call) + " failed: " +             \
                               api_->GetErrorString(r_));                     \
  } while (0)

bool NcclType(DataType t, ncclDataType_t* out) {
  switch (t) {
  case DataType::UINT8:
  case DataType::BOOL: *out = ncclUint8; return true;
  case DataType::INT8: *out = ncclInt8; return true;
  case DataType::INT32: *out = ncclInt32; return true;
  case DataType::INT64: *out = ncclInt64; return true;
  case DataType::FLOAT16: *out = ncclFloat16; return true;
  case DataType::FLOAT32: *out = ncclFloat32; return true;
  case DataType::FLOAT64: *out = ncclFloat64; return true;
  case DataType::BFLOAT16: *out = ncclBfloat16; return true;
  default: return false;
  }
}

ncclRedOp_t NcclOp(ReduceOp op, DataType t) {
  if (t == DataType::BOOL)
    return (op == ReduceOp::MIN || op == ReduceOp::PRODUCT) ? ncclMin : ncclMax;
  switch (op) {
  case ReduceOp::MIN: return ncclMin;
  case ReduceOp::MAX: return ncclMax;
  case ReduceOp::PRODUCT: return ncclProd;
  default: return ncclSum;
  }
}

}  // namespace

NcclOps::NcclOps(GpuOps& gpu)
    : gpu_(gpu),
      buffers_(
          [](size_t n) {
            void* p = nullptr;
            HVD_CUDA(cudaMalloc(&p, std::max<size_t>(n, 256)));
            return p;
          },
          [](void* p) { cudaFree(p); }) {
  std::string err;
  api_ = LoadNccl(&err);
  if (api_ == nullptr) HVD_LOG(WARNING) << "NCCL path unavailable: " << err;
  comms_.set_api(api_);
}

NcclOps::~NcclOps() { Shutdown(); }

void NcclOps::Shutdown() {
  comms_.DestroyAll();
  buffers_.Clear();
}

void* NcclOps::CommFor(ProcessSet& ps) { return CommOver(ps.id, ps.comm); }

void* NcclOps::CommOver(int32_t key, Comm& over) {
  if (void* cached = comms_.Find(key)) return cached;
  // Rank 0 of the group creates the id; it travels over the control plane.
  ncclUniqueId id;
  std::memset(&id, 0, sizeof(id));
  if (over.rank() == 0) HVD_NCCL(api_->GetUniqueId(&id));
  over.Bcast(&id, sizeof(id), 0);
  ncclComm_t comm = nullptr;
  HVD_NCCL(api_->CommInitRank(&comm, over.size(), id, over.rank()));
  over.Barrier();
  comms_.Put(key, comm);
  return comm;
}

bool NcclOps::UseHierarchicalAllreduce(const ProcessSet& ps) const {
  GlobalState& s = gpu_.state();
  return ps.id == 0 && s.hierarchy_usable && s.parameter_manager.HierarchicalAllreduce();
}

// The persistent device fusion buffer, sized for the fusion threshold in
// effect (at least 64 MiB) or for the request if that is larger.
void* NcclOps::Fusion(size_t bytes) {
  const size_t threshold = std::max<size_t>(
      64u << 20, static_cast<size_t>(std::max<int64_t>(
                     0, gpu_.state().parameter_manager.TensorFusionThresholdBytes())));
  return buffers_.Get(gpu_.device(), 0, bytes, threshold, [this] {
    cudaStreamSynchronize(gpu_.stream());
  });
}

Status NcclOps::Execute(std::vector<TensorTableEntry>& entries,
                        const Response& response, ProcessSet& ps) {
  if (api_ == nullptr)
    return Status::PreconditionError(
        "This collective needs NCCL (symmetric memory is not usable for it) "
        "but libnccl.so.2 could not be loaded.");
  if (comms_.failed())
    return Status::UnknownError(
        "NCCL communicators were aborted after an asynchronous error; the job has to "
        "re-initialise (hvd.shutdown() / hvd.init(), which elastic jobs do by themselves).");
  // No abort while this response's calls are being issued.
  std::lock_guard<std::mutex> issuing(comms_.issue_mutex());
  void* comm = CommFor(ps);
  gpu_.WaitForInputs(entries);
  switch (response.type) {
  case Response::ALLREDUCE:
    hierarchical_ = UseHierarchicalAllreduce(ps);
    return Allreduce(entries, response, comm);
  case Response::BROADCAST: return Broadcast(entries, comm);
  case Response::ALLGATHER: return Allgather(entries, response, ps, comm);
  case Response::ALLTOALL: return Alltoall(entries, response, ps, comm);
  case Response::REDUCESCATTER: return Reducescatter(entries, ps, comm);
  case Response::ADASUM: {
    // What the reference's GPU Adasum computes when all ranks share a node
    // (horovod/common/ops/adasum_gpu_operations.cc:64-320 with start_level =
    // local_size; horovod/common/operations.cc:1404-1410 folds 1/local_size
    // into the postscale): an NCCL sum divided by the number of ranks, no
    // Adasum arithmetic. Kept as the baseline of the device Adasum kernels.
    if (gpu_.state().config.local_size != gpu_.state().config.size)
      return Status::PreconditionError(
          "Adasum on CUDA tensors across nodes is not supported on the NCCL path.");
    Response avg = response;
    avg.type = Response::ALLREDUCE;
    avg.reduce_op = ReduceOp::SUM;
    avg.postscale = response.postscale / static_cast<double>(ps.ranks().size());
    hierarchical_ = false;
    return Allreduce(entries, avg, comm);
  }
  default:
    return Status::InvalidArgument("unsupported NCCL collective");
  }
}

Status NcclOps::Allreduce(std::vector<TensorTableEntry>& entries,
                          const Response& response, void* comm_v) {
  ncclComm_t comm = static_cast<ncclComm_t>(comm_v);
  cudaStream_t stream = gpu_.stream();
  Timeline& tl = gpu_.state().timeline;
  ncclDataType_t nt;
  const DataType dtype = response.dtype;
  // fp32 tensors may travel as fp16/bf16: the cast happens in pack/unpack.
  const DataType wire = response.wire_dtype;
  if (!NcclType(wire, &nt))
    return Status::InvalidArgument(std::string("NCCL cannot reduce dtype ") +
                                   DataTypeName(wire));
  const ncclRedOp_t op = NcclOp(response.reduce_op, response.dtype);
  const int64_t es = static_cast<int64_t>(DataTypeSize(wire));

  if (!hierarchical_ && wire == dtype && entries.size() == 1 && entries[0].input &&
      entries[0].output) {
    TensorTableEntry& e = entries[0];
    const void* src = e.input;
    if (response.prescale != 1.0) {
      kern::LaunchScaleBuffer(e.input, e.output, e.num_elements(), dtype,
                              response.prescale, stream);
      src = e.output;
    }
    gpu_.ActStart(e.name, HVD_ACT_NCCL_ALLREDUCE);
    HVD_NCCL(api_->AllReduce(src, e.output, e.num_elements(), nt, op, comm, stream));
    gpu_.ActEnd(e.name);
    if (response.postscale != 1.0)
      kern::LaunchScaleBuffer(e.output, e.output, e.num_elements(), dtype,
                              response.postscale, stream);
    return gpu_.Complete(entries);
  }

  // Fused: pack(+prescale) -> ncclAllReduce -> unpack(+postscale).
  const int64_t align = FUSION_ALIGN_BYTES / es;
  const size_t n = entries.size();
  DescriptorRing::Slot slot = gpu_.ring().Acquire();
  int64_t *d_off, *d_cnt;
  const void** d_in;
  void** d_out;
  int64_t* h_off = slot.Alloc<int64_t>(n + 1, &d_off);
  int64_t* h_cnt = slot.Alloc<int64_t>(n, &d_cnt);
  const void** h_in = slot.Alloc<const void*>(n, &d_in);
  void** h_out = slot.Alloc<void*>(n, &d_out);
  if (!h_off || !h_cnt || !h_in || !h_out)
    return Status::UnknownError("descriptor slot too small");
  int64_t off = 0;
  for (size_t i = 0; i < n; ++i) {
    h_off[i] = off;
    h_cnt[i] = entries[i].num_elements();
    h_in[i] = entries[i].input;
    h_out[i] = entries[i].output;
    off += RoundUp(h_cnt[i], align);
  }
  h_off[n] = off;
  gpu_.ring().Commit(slot, stream);
  kern::TensorList list = {static_cast<int>(n), d_off, d_cnt, d_in, d_out};
  // The hierarchical variant cuts the buffer into local_size equal shards.
  GlobalState& gs = gpu_.state();
  const int64_t local = hierarchical_ ? gs.local_comm.size() : 1;
  const int64_t padded = RoundUp(off, local * align);
  void* buf = Fusion(static_cast<size_t>(padded * es));
  if (padded > off)
    HVD_CUDA(cudaMemsetAsync(static_cast<char*>(buf) + off * es, 0,
                             static_cast<size_t>((padded - off) * es), stream));
  gpu_.ActStart(entries, HVD_ACT_MEMCPY_IN_FUSION_BUFFER);
  host_trace::Mark("plan");
  kern::LaunchPackUnpack(list, dtype, wire, buf, response.prescale, true, off, stream);
  host_trace::Mark("pack launch");
  gpu_.ActEnd(entries);
  gpu_.ActStart(entries, HVD_ACT_NCCL_ALLREDUCE);
  if (hierarchical_) {
    // Reduce-scatter inside the host, allreduce of each rank's shard across
    // hosts, allgather inside the host
    // (horovod/common/ops/nccl_operations.cc:233-440; the cross-host step is
    // an NCCL allreduce here instead of a copy to the host and MPI).
    ncclComm_t lc = static_cast<ncclComm_t>(CommOver(-1, gs.local_comm));
    ncclComm_t cc = static_cast<ncclComm_t>(CommOver(-2, gs.cross_comm));
    const int64_t shard = padded / local;
    char* mine = static_cast<char*>(buf) + gs.local_comm.rank() * shard * es;
    HVD_NCCL(api_->ReduceScatter(buf, mine, shard, nt, op, lc, stream));
    HVD_NCCL(api_->AllReduce(mine, mine, shard, nt, op, cc, stream));
    HVD_NCCL(api_->AllGather(mine, buf, shard, nt, lc, stream));
  } else {
    HVD_NCCL(api_->AllReduce(buf, buf, off, nt, op, comm, stream));
  }
  host_trace::Mark("nccl call");
  gpu_.ActEnd(entries);
  gpu_.ActStart(entries, HVD_ACT_MEMCPY_OUT_FUSION_BUFFER);
  kern::LaunchPackUnpack(list, dtype, wire, buf, response.postscale, false, off, stream);
  host_trace::Mark("unpack launch");
  gpu_.ActEnd(entries);
  gpu_.ring().Release(slot, stream);
  return gpu_.Complete(entries);
}

}  // namespace hvd
