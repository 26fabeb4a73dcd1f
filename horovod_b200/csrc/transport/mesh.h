// CPU control/data plane: a full mesh of TCP connections between the ranks of
// a job, and `Comm`, a communicator over any subset of those ranks that
// implements the collectives the controller and the CPU ops need.
//
// This replaces the reference's Gloo/MPI contexts and controllers
// (horovod/common/gloo/gloo_context.cc:134-232, gloo_controller.cc:116-305,
// horovod/common/mpi/mpi_controller.cc:28-271) with one socket layer that has
// no third-party dependency. All sockets are non-blocking and every wait is a
// poll() with a deadline, so a dead or silent peer surfaces as an exception
// (which the background loop turns into HorovodInternalError), never a hang.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "../common/common.h"

namespace hvd {

class TransportError : public std::runtime_error {
public:
  explicit TransportError(const std::string& m) : std::runtime_error(m) {}
};

class TcpMesh {
public:
  TcpMesh() = default;
  ~TcpMesh() { Close(); }
  TcpMesh(const TcpMesh&) = delete;
  TcpMesh& operator=(const TcpMesh&) = delete;

  // Opens the listening socket on an ephemeral port and returns the
  // "host:port" string other ranks connect to. `advertise_host` is the
  // address peers can reach this process at.
  std::string Listen(const std::string& advertise_host);
  // Builds the mesh: connects to every lower rank, accepts every higher one.
  // addrs[i] is what rank i returned from Listen(). `token` must match on
  // both ends (guards against stray connections from an earlier job).
  void Connect(int rank, int size, const std::vector<std::string>& addrs,
               uint64_t token, double timeout_s);
  void Close();

  int rank() const { return rank_; }
  int size() const { return size_; }
  void set_timeout(double s) { timeout_s_ = s; }
  double timeout() const { return timeout_s_; }

  void Send(int peer, const void* buf, size_t len);
  void Recv(int peer, void* buf, size_t len);
  // Full-duplex exchange that cannot deadlock on full socket buffers.
  // Either side may be a null transfer (len 0).
  void SendRecv(int send_peer, const void* sbuf, size_t slen, int recv_peer,
                void* rbuf, size_t rlen);

private:
  int rank_ = 0;
  int size_ = 1;
  int listen_fd_ = -1;
  double timeout_s_ = 30.0;
  std::vector<int> fds_;  // fds_[peer], -1 for self
};

// Communicator over `ranks` (global mesh ranks, ascending). rank()/size() and
// every root argument are relative to that list.
class Comm {
public:
  Comm() = default;
  Comm(TcpMesh* mesh, std::vector<int> ranks);

  int rank() const { return rank_; }
  int size() const { return static_cast<int>(ranks_.size()); }
  const std::vector<int>& global_ranks() const { return ranks_; }
  bool contains_me() const { return rank_ >= 0; }
  // Communicator over some of this communicator's ranks (given relative to
  // this communicator, ascending).
  Comm Subset(const std::vector<int>& members) const {
    std::vector<int> global;
    for (int m : members) global.push_back(ranks_[m]);
    return Comm(mesh_, std::move(global));
  }

  void Barrier();
  void Bcast(void* buf, size_t len, int root);
  // Length-prefixed variable-size blob broadcast.
  void BcastBlob(std::string* blob, int root);
  // Root receives one blob per rank (its own included, in rank order).
  void GatherBlobs(const std::string& mine, int root,
                   std::vector<std::string>* out);
  // Element-wise AND / OR over 64-bit words, result on every rank.
  void AllreduceBits(uint64_t* words, size_t n, bool bitwise_and);
  // Fixed-size allgather: recv holds size()*len bytes.
  void Allgather(const void* send, size_t len, void* recv);
  // Variable-size allgather: block r has lens[r] bytes at offset sum(lens[<r]).
  void Allgatherv(const void* send, const std::vector<int64_t>& lens,
                  void* recv);
  // send/recv blocks are ordered by peer rank; byte counts per peer.
  void Alltoallv(const void* send, const std::vector<int64_t>& send_lens,
                 void* recv, const std::vector<int64_t>& recv_lens);
  // In-place typed reduction. op is SUM, MIN, MAX or PRODUCT.
  void Allreduce(void* buf, int64_t count, DataType dtype, ReduceOp op);
  // Point-to-point inside the communicator (used by the CPU Adasum).
  void SendRecv(int send_peer, const void* sbuf, size_t slen, int recv_peer,
                void* rbuf, size_t rlen);

private:
  int g(int r) const { return ranks_[r]; }
  TcpMesh* mesh_ = nullptr;
  std::vector<int> ranks_;
  int rank_ = -1;
};

// dst[i] = dst[i] (op) src[i] for every supported dtype; fp16/bf16 are
// accumulated through fp32 (F16C vector path for fp16 when the CPU has it).
// Parity: horovod/common/half.cc:44-76 (custom fp16 sum).
void ReduceInto(void* dst, const void* src, int64_t count, DataType dtype,
                ReduceOp op);
// buf[i] *= factor (floating types scale in double/float; integers scale in
// double and truncate like the framework's integer division).
// Parity: horovod/common/ops/collective_operations.h:91-127.
void ScaleBufferCPU(void* buf, int64_t count, DataType dtype, double factor);

}  // namespace hvd
