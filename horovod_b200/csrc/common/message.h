// Negotiation messages exchanged by the controllers every cycle, with a
// compact little-endian binary encoding (no schema compiler needed).
//
// Parity: horovod/common/message.h:50-252 and the FlatBuffers schema in
// horovod/common/wire/message.fbs:18-119. Extra over that snapshot: a
// REDUCESCATTER request type, a reduce_op field (so MIN/MAX/PRODUCT can be
// validated across ranks) and the BFLOAT16 dtype id.
#pragma once

#include <stdexcept>
#include <string>
#include <vector>

#include "common.h"

namespace hvd {

// Append-only byte writer / bounds-checked reader used by the wire format.
class WireWriter {
public:
  void u8(uint8_t v) { buf_.push_back(static_cast<char>(v)); }
  void i32(int32_t v) { raw(&v, 4); }
  void i64(int64_t v) { raw(&v, 8); }
  void f64(double v) { raw(&v, 8); }
  void str(const std::string& s) {
    i32(static_cast<int32_t>(s.size()));
    raw(s.data(), s.size());
  }
  void raw(const void* p, size_t n) {
    const char* c = static_cast<const char*>(p);
    buf_.insert(buf_.end(), c, c + n);
  }
  std::string& buffer() { return buf_; }

private:
  std::string buf_;
};

class WireReader {
public:
  WireReader(const char* p, size_t n) : p_(p), end_(p + n) {}
  uint8_t u8() { uint8_t v; raw(&v, 1); return v; }
  int32_t i32() { int32_t v; raw(&v, 4); return v; }
  int64_t i64() { int64_t v; raw(&v, 8); return v; }
  double f64() { double v; raw(&v, 8); return v; }
  std::string str() {
    int32_t n = i32();
    check(n >= 0 && static_cast<size_t>(n) <= remaining());
    std::string s(p_, p_ + n);
    p_ += n;
    return s;
  }
  void raw(void* out, size_t n) {
    check(n <= remaining());
    std::memcpy(out, p_, n);
    p_ += n;
  }
  size_t remaining() const { return static_cast<size_t>(end_ - p_); }
  bool failed() const { return failed_; }

private:
  void check(bool ok) {
    if (!ok) {
      failed_ = true;
      throw std::runtime_error("hvd wire: truncated or corrupt message");
    }
  }
  const char* p_;
  const char* end_;
  bool failed_ = false;
};

class Request {
public:
  enum Type : uint8_t {
    ALLREDUCE = 0,
    ALLGATHER = 1,
    BROADCAST = 2,
    JOIN = 3,
    ADASUM = 4,
    ALLTOALL = 5,
    REDUCESCATTER = 6,
  };
  static const char* TypeName(Type t);

  int32_t request_rank = 0;  // rank inside the process set
  Type type = ALLREDUCE;
  DataType dtype = DataType::FLOAT32;
  std::string name;
  int32_t root_rank = 0;
  int32_t device = CPU_DEVICE_ID;
  int32_t group_id = -1;
  ReduceOp reduce_op = ReduceOp::SUM;
  std::vector<int64_t> shape;
  double prescale = 1.0;
  double postscale = 1.0;
  // Element type on the wire (fp32 tensors may travel as fp16/bf16, cast
  // inside the collective kernel); equals dtype when there is no cast.
  DataType wire_dtype = DataType::FLOAT32;

  void Serialize(WireWriter& w) const;
  static Request Parse(WireReader& r);
};

class RequestList {
public:
  std::vector<Request> requests;
  bool shutdown = false;

  std::string Serialize() const;
  static RequestList Parse(const char* data, size_t len);
};

class Response {
public:
  enum Type : uint8_t {
    ALLREDUCE = 0,
    ALLGATHER = 1,
    BROADCAST = 2,
    JOIN = 3,
    ADASUM = 4,
    ALLTOALL = 5,
    REDUCESCATTER = 6,
    ERROR = 7,
  };
  static const char* TypeName(Type t);

  Type type = ALLREDUCE;
  std::vector<std::string> names;
  std::string error_message;
  std::vector<int32_t> devices;
  // ALLREDUCE/ADASUM/REDUCESCATTER: element count per tensor.
  // ALLGATHER: for each tensor, the dim-0 size of every rank (size entries
  // per tensor, tensor-major).
  std::vector<int64_t> tensor_sizes;
  DataType dtype = DataType::FLOAT32;
  ReduceOp reduce_op = ReduceOp::SUM;
  double prescale = 1.0;
  double postscale = 1.0;
  int32_t last_joined_rank = -1;
  int32_t root_rank = 0;  // BROADCAST only
  DataType wire_dtype = DataType::FLOAT32;  // reductions only

  void add_name(const std::string& n) { names.push_back(n); }
  std::string names_string() const;
  void Serialize(WireWriter& w) const;
  static Response Parse(WireReader& r);
};

class ResponseList {
public:
  std::vector<Response> responses;
  bool shutdown = false;

  std::string Serialize() const;
  static ResponseList Parse(const char* data, size_t len);
};

// An ALLTOALL response whose ranks all left the splits to the library (even
// split) carries every rank's first dimension, so that every rank knows the
// whole split table: rank r sends rows[r] rows to each peer. Returns false
// when the ranks passed explicit splits and have to exchange them.
inline bool AlltoallEvenRows(const Response& response, int ranks, std::vector<int32_t>* rows) {
  if (response.type != Response::ALLTOALL || response.root_rank != 1 ||
      response.names.size() != 1 || static_cast<int>(response.tensor_sizes.size()) != ranks)
    return false;
  rows->resize(ranks);
  for (int r = 0; r < ranks; ++r) {
    if (response.tensor_sizes[r] % ranks != 0) return false;
    (*rows)[r] = static_cast<int32_t>(response.tensor_sizes[r] / ranks);
  }
  return true;
}

}  // namespace hvd
