// Core value types shared by every layer of the runtime: status codes, data
// types, reduce ops, tensor shapes and the table entry that describes one
// pending collective.
//
// Parity: horovod/common/common.h:158-379 (Status, TensorShape, ReadyEvent,
// OpContext, TensorTableEntry) and horovod/common/message.h:30-41 (DataType).
// The layout here is different: entries carry raw pointers plus an opaque
// framework context, so the core never includes framework headers.
#pragma once

#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace hvd {

// Wire ids are stable: BFLOAT16 is appended after BOOL.
enum class DataType : uint8_t {
  UINT8 = 0,
  INT8 = 1,
  UINT16 = 2,
  INT16 = 3,
  INT32 = 4,
  INT64 = 5,
  FLOAT16 = 6,
  FLOAT32 = 7,
  FLOAT64 = 8,
  BOOL = 9,
  BFLOAT16 = 10,
};

inline size_t DataTypeSize(DataType t) {
  switch (t) {
  case DataType::UINT8:
  case DataType::INT8:
  case DataType::BOOL:
    return 1;
  case DataType::UINT16:
  case DataType::INT16:
  case DataType::FLOAT16:
  case DataType::BFLOAT16:
    return 2;
  case DataType::INT32:
  case DataType::FLOAT32:
    return 4;
  case DataType::INT64:
  case DataType::FLOAT64:
    return 8;
  }
  return 0;
}

inline const char* DataTypeName(DataType t) {
  switch (t) {
  case DataType::UINT8: return "uint8";
  case DataType::INT8: return "int8";
  case DataType::UINT16: return "uint16";
  case DataType::INT16: return "int16";
  case DataType::INT32: return "int32";
  case DataType::INT64: return "int64";
  case DataType::FLOAT16: return "float16";
  case DataType::FLOAT32: return "float32";
  case DataType::FLOAT64: return "float64";
  case DataType::BOOL: return "bool";
  case DataType::BFLOAT16: return "bfloat16";
  }
  return "<unknown>";
}

inline bool IsFloatingPoint(DataType t) {
  return t == DataType::FLOAT16 || t == DataType::FLOAT32 ||
         t == DataType::FLOAT64 || t == DataType::BFLOAT16;
}

// Numeric values are part of the Python API (hvd.Average == 0 ...).
enum class ReduceOp : uint8_t {
  AVERAGE = 0,
  SUM = 1,
  ADASUM = 2,
  MIN = 3,
  MAX = 4,
  PRODUCT = 5,
};

inline const char* ReduceOpName(ReduceOp op) {
  switch (op) {
  case ReduceOp::AVERAGE: return "average";
  case ReduceOp::SUM: return "sum";
  case ReduceOp::ADASUM: return "adasum";
  case ReduceOp::MIN: return "min";
  case ReduceOp::MAX: return "max";
  case ReduceOp::PRODUCT: return "product";
  }
  return "<unknown>";
}

constexpr int CPU_DEVICE_ID = -1;

// Every tensor inside a fused buffer starts on this boundary so that vector
// loads and stores never straddle two tensors.
constexpr int64_t FUSION_ALIGN_BYTES = 16;
// The fusion threshold is rounded up to a multiple of local_size * this unit
// so that every rank's shard of a full buffer is 512-byte aligned.
constexpr int64_t FUSION_ATOMIC_UNIT = 64 * 8;

enum class StatusType {
  OK,
  UNKNOWN_ERROR,
  PRECONDITION_ERROR,
  ABORTED,
  INVALID_ARGUMENT,
  IN_PROGRESS,
};

class Status {
public:
  Status() = default;
  static Status OK() { return Status(); }
  static Status UnknownError(std::string m) {
    return Status(StatusType::UNKNOWN_ERROR, std::move(m));
  }
  static Status PreconditionError(std::string m) {
    return Status(StatusType::PRECONDITION_ERROR, std::move(m));
  }
  static Status Aborted(std::string m) {
    return Status(StatusType::ABORTED, std::move(m));
  }
  static Status InvalidArgument(std::string m) {
    return Status(StatusType::INVALID_ARGUMENT, std::move(m));
  }
  static Status InProgress() { return Status(StatusType::IN_PROGRESS, ""); }
  bool ok() const { return type_ == StatusType::OK; }
  bool in_progress() const { return type_ == StatusType::IN_PROGRESS; }
  StatusType type() const { return type_; }
  const std::string& reason() const { return reason_; }

private:
  Status(StatusType t, std::string m) : type_(t), reason_(std::move(m)) {}
  StatusType type_ = StatusType::OK;
  std::string reason_;
};

// Messages surfaced to every pending callback when the runtime goes down.
extern const char* const SHUT_DOWN_ERROR_MESSAGE;
extern const char* const DUPLICATE_NAME_ERROR_MESSAGE;

class TensorShape {
public:
  TensorShape() = default;
  explicit TensorShape(std::vector<int64_t> d) : dims_(std::move(d)) {}
  void AddDim(int64_t d) { dims_.push_back(d); }
  int dims() const { return static_cast<int>(dims_.size()); }
  int64_t dim_size(int i) const { return dims_[i]; }
  int64_t num_elements() const {
    int64_t n = 1;
    for (auto d : dims_) n *= d;
    return n;
  }
  const std::vector<int64_t>& to_vector() const { return dims_; }
  std::string DebugString() const {
    std::ostringstream s;
    s << "[";
    for (size_t i = 0; i < dims_.size(); ++i) {
      if (i) s << ", ";
      s << dims_[i];
    }
    s << "]";
    return s.str();
  }
  bool operator==(const TensorShape& o) const { return dims_ == o.dims_; }
  bool operator!=(const TensorShape& o) const { return dims_ != o.dims_; }

private:
  std::vector<int64_t> dims_;
};

// Marks the point on the producer's stream after which the input is valid.
// CPU tensors have no ready event.
class ReadyEvent {
public:
  virtual ~ReadyEvent() = default;
  // True once the producer work has finished on the device.
  virtual bool Ready() const = 0;
  // Makes `stream` (a cudaStream_t) wait for the producer without blocking
  // the host.
  virtual void StreamWait(void* stream) const = 0;
};

// Framework services an op may need after negotiation: output allocation for
// ops whose result size depends on other ranks, and zero tensors for ranks
// that have joined.
class OpContext {
public:
  virtual ~OpContext() = default;
  // Allocates the op's output with the given shape on the entry's device and
  // returns its data pointer. `stream` is the stream the collective runs on
  // (nullptr for CPU) so the allocation can be tied to it.
  virtual Status AllocateOutput(const TensorShape& shape, void* stream,
                                void** data) = 0;
  // For alltoall: hands the received splits back to the framework.
  virtual void SetReceivedSplits(const std::vector<int32_t>& splits) {}
};

// Completion information given to the framework callback. `done_event`
// wraps a cudaEvent_t recorded on the communication stream after the op's
// last kernel (null for CPU ops or host-synchronised completion); the event
// goes back to its pool when the last holder drops the pointer.
struct Completion {
  Status status;
  std::shared_ptr<void> done_event;
};

using StatusCallback = std::function<void(const Completion&)>;

struct TensorTableEntry {
  std::string name;
  const void* input = nullptr;
  void* output = nullptr;
  TensorShape shape;
  DataType dtype = DataType::FLOAT32;
  // Element type on the wire for reductions (set equal to dtype unless the
  // caller asked for a 16-bit wire format for fp32 data).
  DataType wire_dtype = DataType::FLOAT32;
  int device = CPU_DEVICE_ID;
  int root_rank = 0;
  ReduceOp reduce_op = ReduceOp::SUM;
  double prescale = 1.0;
  double postscale = 1.0;
  std::vector<int32_t> splits;  // alltoall send splits (dim 0 rows per peer)
  int32_t process_set_id = 0;
  int32_t group_id = -1;
  std::shared_ptr<OpContext> context;
  std::shared_ptr<ReadyEvent> ready;
  StatusCallback callback;
  // Start of the op in steady-clock microseconds (timeline, stall check).
  int64_t enqueue_us = 0;

  int64_t num_elements() const { return shape.num_elements(); }
  int64_t size_bytes() const {
    return shape.num_elements() * static_cast<int64_t>(DataTypeSize(dtype));
  }
  void Finish(const Status& s,
              const std::shared_ptr<void>& done_event = nullptr) const {
    if (callback) {
      Completion c;
      c.status = s;
      c.done_event = done_event;
      callback(c);
    }
  }
};

int64_t NowMicros();

// Pins the calling thread to one CPU core (HOROVOD_THREAD_AFFINITY); a
// negative core leaves the thread alone.
void SetThreadAffinity(int core);
// The core that a HOROVOD_THREAD_AFFINITY value names for `local_rank`, or -1.
int AffinityCore(const std::string& spec, int local_rank);

inline int64_t RoundUp(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

}  // namespace hvd
