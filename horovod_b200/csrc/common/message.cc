#include "message.h"

#include <stdexcept>

namespace hvd {

const char* Request::TypeName(Type t) {
  switch (t) {
  case ALLREDUCE: return "ALLREDUCE";
  case ALLGATHER: return "ALLGATHER";
  case BROADCAST: return "BROADCAST";
  case JOIN: return "JOIN";
  case ADASUM: return "ADASUM";
  case ALLTOALL: return "ALLTOALL";
  case REDUCESCATTER: return "REDUCESCATTER";
  }
  return "<unknown>";
}

const char* Response::TypeName(Type t) {
  switch (t) {
  case ALLREDUCE: return "ALLREDUCE";
  case ALLGATHER: return "ALLGATHER";
  case BROADCAST: return "BROADCAST";
  case JOIN: return "JOIN";
  case ADASUM: return "ADASUM";
  case ALLTOALL: return "ALLTOALL";
  case REDUCESCATTER: return "REDUCESCATTER";
  case ERROR: return "ERROR";
  }
  return "<unknown>";
}

void Request::Serialize(WireWriter& w) const {
  w.i32(request_rank);
  w.u8(type);
  w.u8(static_cast<uint8_t>(dtype));
  w.str(name);
  w.i32(root_rank);
  w.i32(device);
  w.i32(group_id);
  w.u8(static_cast<uint8_t>(reduce_op));
  w.i32(static_cast<int32_t>(shape.size()));
  for (auto d : shape) w.i64(d);
  w.f64(prescale);
  w.f64(postscale);
  w.u8(static_cast<uint8_t>(wire_dtype));
}

Request Request::Parse(WireReader& r) {
  Request q;
  q.request_rank = r.i32();
  q.type = static_cast<Type>(r.u8());
  q.dtype = static_cast<DataType>(r.u8());
  q.name = r.str();
  q.root_rank = r.i32();
  q.device = r.i32();
  q.group_id = r.i32();
  q.reduce_op = static_cast<ReduceOp>(r.u8());
  int32_t nd = r.i32();
  if (nd < 0 || nd > 64) throw std::runtime_error("hvd wire: bad rank");
  q.shape.resize(nd);
  for (auto& d : q.shape) d = r.i64();
  q.prescale = r.f64();
  q.postscale = r.f64();
  q.wire_dtype = static_cast<DataType>(r.u8());
  return q;
}

std::string RequestList::Serialize() const {
  WireWriter w;
  w.u8(shutdown ? 1 : 0);
  w.i32(static_cast<int32_t>(requests.size()));
  for (auto& q : requests) q.Serialize(w);
  return std::move(w.buffer());
}

RequestList RequestList::Parse(const char* data, size_t len) {
  WireReader r(data, len);
  RequestList l;
  l.shutdown = r.u8() != 0;
  int32_t n = r.i32();
  if (n < 0) throw std::runtime_error("hvd wire: bad request count");
  l.requests.reserve(n);
  for (int32_t i = 0; i < n; ++i) l.requests.push_back(Request::Parse(r));
  return l;
}

std::string Response::names_string() const {
  std::string s;
  for (size_t i = 0; i < names.size(); ++i) {
    if (i) s += ", ";
    s += names[i];
  }
  return s;
}

void Response::Serialize(WireWriter& w) const {
  w.u8(type);
  w.i32(static_cast<int32_t>(names.size()));
  for (auto& n : names) w.str(n);
  w.str(error_message);
  w.i32(static_cast<int32_t>(devices.size()));
  for (auto d : devices) w.i32(d);
  w.i32(static_cast<int32_t>(tensor_sizes.size()));
  for (auto s : tensor_sizes) w.i64(s);
  w.u8(static_cast<uint8_t>(dtype));
  w.u8(static_cast<uint8_t>(reduce_op));
  w.f64(prescale);
  w.f64(postscale);
  w.i32(last_joined_rank);
  w.i32(root_rank);
  w.u8(static_cast<uint8_t>(wire_dtype));
}

Response Response::Parse(WireReader& r) {
  Response p;
  p.type = static_cast<Type>(r.u8());
  int32_t n = r.i32();
  if (n < 0) throw std::runtime_error("hvd wire: bad name count");
  p.names.reserve(n);
  for (int32_t i = 0; i < n; ++i) p.names.push_back(r.str());
  p.error_message = r.str();
  n = r.i32();
  if (n < 0) throw std::runtime_error("hvd wire: bad device count");
  p.devices.resize(n);
  for (auto& d : p.devices) d = r.i32();
  n = r.i32();
  if (n < 0) throw std::runtime_error("hvd wire: bad size count");
  p.tensor_sizes.resize(n);
  for (auto& s : p.tensor_sizes) s = r.i64();
  p.dtype = static_cast<DataType>(r.u8());
  p.reduce_op = static_cast<ReduceOp>(r.u8());
  p.prescale = r.f64();
  p.postscale = r.f64();
  p.last_joined_rank = r.i32();
  p.root_rank = r.i32();
  p.wire_dtype = static_cast<DataType>(r.u8());
  return p;
}

std::string ResponseList::Serialize() const {
  WireWriter w;
  w.u8(shutdown ? 1 : 0);
  w.i32(static_cast<int32_t>(responses.size()));
  for (auto& p : responses) p.Serialize(w);
  return std::move(w.buffer());
}

ResponseList ResponseList::Parse(const char* data, size_t len) {
  WireReader r(data, len);
  ResponseList l;
  l.shutdown = r.u8() != 0;
  int32_t n = r.i32();
  if (n < 0) throw std::runtime_error("hvd wire: bad response count");
  l.responses.reserve(n);
  for (int32_t i = 0; i < n; ++i) l.responses.push_back(Response::Parse(r));
  return l;
}

}  // namespace hvd
