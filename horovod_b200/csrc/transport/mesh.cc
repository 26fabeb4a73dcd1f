#include "mesh.h"

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>

#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include "../common/cpu_vector.h"
#include "../common/half.h"
#include "../common/logging.h"

namespace hvd {

namespace {

using Clock = std::chrono::steady_clock;

double Since(Clock::time_point t0) {
  return std::chrono::duration<double>(Clock::now() - t0).count();
}

void SetNonBlocking(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
}

void TuneSocket(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int buf = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

[[noreturn]] void Fail(const std::string& what) {
  throw TransportError("hvd transport: " + what);
}

// Waits until fd is readable/writable or the deadline passes.
void WaitFd(int fd, short events, Clock::time_point t0, double timeout_s,
            const char* what, int peer) {
  for (;;) {
    double left = timeout_s - Since(t0);
    if (left <= 0)
      Fail(std::string("timed out after ") + std::to_string(timeout_s) +
           " s waiting to " + what + " rank " + std::to_string(peer));
    struct pollfd p = {fd, events, 0};
    int r = poll(&p, 1, static_cast<int>(std::min(left, 1.0) * 1000) + 1);
    if (r < 0) {
      if (errno == EINTR) continue;
      Fail(std::string("poll failed: ") + std::strerror(errno));
    }
    if (r > 0) return;  // readable, writable, or error (next syscall reports)
  }
}

struct HostPort {
  std::string host;
  int port;
};

HostPort SplitAddr(const std::string& a) {
  auto pos = a.rfind(':');
  if (pos == std::string::npos) Fail("bad address '" + a + "'");
  return {a.substr(0, pos), std::atoi(a.c_str() + pos + 1)};
}

int ConnectTo(const HostPort& hp, double timeout_s) {
  auto t0 = Clock::now();
  std::string last_err = "unknown";
  while (Since(t0) < timeout_s) {
    struct addrinfo hints;
    std::memset(&hints, 0, sizeof(hints));
    hints.ai_family = AF_UNSPEC;
    hints.ai_socktype = SOCK_STREAM;
    struct addrinfo* res = nullptr;
    std::string port = std::to_string(hp.port);
    int rc = getaddrinfo(hp.host.c_str(), port.c_str(), &hints, &res);
    if (rc != 0) {
      last_err = gai_strerror(rc);
    } else {
      for (auto* ai = res; ai != nullptr; ai = ai->ai_next) {
        int fd = socket(ai->ai_family, ai->ai_socktype, ai->ai_protocol);
        if (fd < 0) continue;
        if (connect(fd, ai->ai_addr, ai->ai_addrlen) == 0) {
          freeaddrinfo(res);
          return fd;
        }
        last_err = std::strerror(errno);
        close(fd);
      }
      freeaddrinfo(res);
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
  Fail("could not connect to " + hp.host + ":" + std::to_string(hp.port) +
       " (" + last_err + ")");
}

void BlockingWrite(int fd, const void* buf, size_t len) {
  const char* p = static_cast<const char*>(buf);
  while (len > 0) {
    ssize_t n = ::send(fd, p, len, MSG_NOSIGNAL);
    if (n < 0) {
      if (errno == EINTR) continue;
      Fail(std::string("handshake send failed: ") + std::strerror(errno));
    }
    p += n;
    len -= static_cast<size_t>(n);
  }
}

bool TimedRead(int fd, void* buf, size_t len, double timeout_s) {
  auto t0 = Clock::now();
  char* p = static_cast<char*>(buf);
  while (len > 0) {
    double left = timeout_s - Since(t0);
    if (left <= 0) return false;
    struct pollfd pf = {fd, POLLIN, 0};
    int r = poll(&pf, 1, static_cast<int>(left * 1000) + 1);
    if (r < 0 && errno == EINTR) continue;
    if (r <= 0) return false;
    ssize_t n = ::recv(fd, p, len, 0);
    if (n == 0) return false;
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return false;
    }
    p += n;
    len -= static_cast<size_t>(n);
  }
  return true;
}

struct Hello {
  uint64_t token;
  int32_t rank;
  int32_t pad;
};

}  // namespace

std::string TcpMesh::Listen(const std::string& advertise_host) {
  if (listen_fd_ >= 0) close(listen_fd_);
  listen_fd_ = socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) Fail("cannot create listening socket");
  int one = 1;
  setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in addr;
  std::memset(&addr, 0, sizeof(addr));
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = 0;
  if (bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0)
    Fail(std::string("bind failed: ") + std::strerror(errno));
  if (listen(listen_fd_, 256) != 0)
    Fail(std::string("listen failed: ") + std::strerror(errno));
  socklen_t alen = sizeof(addr);
  getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&addr), &alen);
  return advertise_host + ":" + std::to_string(ntohs(addr.sin_port));
}

void TcpMesh::Connect(int rank, int size, const std::vector<std::string>& addrs,
                      uint64_t token, double timeout_s) {
  rank_ = rank;
  size_ = size;
  fds_.assign(size, -1);
  if (static_cast<int>(addrs.size()) != size) Fail("address list size mismatch");
  // Lower ranks are dialled, higher ranks dial us.
  for (int peer = 0; peer < rank; ++peer) {
    int fd = ConnectTo(SplitAddr(addrs[peer]), timeout_s);
    Hello h = {token, rank, 0};
    BlockingWrite(fd, &h, sizeof(h));
    fds_[peer] = fd;
  }
  auto t0 = Clock::now();
  int expected = size - 1 - rank;
  while (expected > 0) {
    double left = timeout_s - Since(t0);
    if (left <= 0)
      Fail("timed out waiting for " + std::to_string(expected) +
           " higher rank(s) to connect");
    struct pollfd pf = {listen_fd_, POLLIN, 0};
    int r = poll(&pf, 1, static_cast<int>(std::min(left, 1.0) * 1000) + 1);
    if (r <= 0) continue;
    int fd = accept(listen_fd_, nullptr, nullptr);
    if (fd < 0) continue;
    Hello h;
    if (!TimedRead(fd, &h, sizeof(h), 5.0) || h.token != token ||
        h.rank <= rank || h.rank >= size || fds_[h.rank] != -1) {
      close(fd);  // stray connection
      continue;
    }
    fds_[h.rank] = fd;
    --expected;
  }
  for (int fd : fds_) {
    if (fd >= 0) {
      TuneSocket(fd);
      SetNonBlocking(fd);
    }
  }
  if (listen_fd_ >= 0) {
    close(listen_fd_);
    listen_fd_ = -1;
  }
}

void TcpMesh::Close() {
  for (int& fd : fds_) {
    if (fd >= 0) {
      shutdown(fd, SHUT_RDWR);
      close(fd);
      fd = -1;
    }
  }
  if (listen_fd_ >= 0) {
    close(listen_fd_);
    listen_fd_ = -1;
  }
}

void TcpMesh::Send(int peer, const void* buf, size_t len) {
  SendRecv(peer, buf, len, -1, nullptr, 0);
}

void TcpMesh::Recv(int peer, void* buf, size_t len) {
  SendRecv(-1, nullptr, 0, peer, buf, len);
}

void TcpMesh::SendRecv(int send_peer, const void* sbuf, size_t slen,
                       int recv_peer, void* rbuf, size_t rlen) {
  const char* sp = static_cast<const char*>(sbuf);
  char* rp = static_cast<char*>(rbuf);
  if (send_peer == rank_ && recv_peer == rank_) {
    if (slen != rlen) Fail("self sendrecv size mismatch");
    if (slen) std::memcpy(rp, sp, slen);
    return;
  }
  if (send_peer == rank_ || recv_peer == rank_) Fail("half self sendrecv");
  int sfd = (send_peer >= 0 && slen > 0) ? fds_.at(send_peer) : -1;
  int rfd = (recv_peer >= 0 && rlen > 0) ? fds_.at(recv_peer) : -1;
  if ((send_peer >= 0 && slen > 0 && sfd < 0) ||
      (recv_peer >= 0 && rlen > 0 && rfd < 0))
    Fail("no connection to peer (mesh closed?)");
  size_t sleft = sfd >= 0 ? slen : 0;
  size_t rleft = rfd >= 0 ? rlen : 0;
  auto t0 = Clock::now();
  while (sleft > 0 || rleft > 0) {
    bool progressed = false;
    if (sleft > 0) {
      ssize_t n = ::send(sfd, sp, sleft, MSG_NOSIGNAL);
      if (n > 0) {
        sp += n;
        sleft -= static_cast<size_t>(n);
        progressed = true;
      } else if (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK &&
                 errno != EINTR) {
        Fail("send to rank " + std::to_string(send_peer) +
             " failed: " + std::strerror(errno));
      }
    }
    if (rleft > 0) {
      ssize_t n = ::recv(rfd, rp, rleft, 0);
      if (n > 0) {
        rp += n;
        rleft -= static_cast<size_t>(n);
        progressed = true;
      } else if (n == 0) {
        Fail("rank " + std::to_string(recv_peer) + " closed the connection");
      } else if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) {
        Fail("recv from rank " + std::to_string(recv_peer) +
             " failed: " + std::strerror(errno));
      }
    }
    if (progressed) {
      t0 = Clock::now();
      continue;
    }
    double left = timeout_s_ - Since(t0);
    if (left <= 0)
      Fail("timed out after " + std::to_string(timeout_s_) +
           " s exchanging data with rank " +
           std::to_string(rleft > 0 ? recv_peer : send_peer));
    struct pollfd pf[2];
    int n = 0;
    if (sleft > 0) pf[n++] = {sfd, POLLOUT, 0};
    if (rleft > 0) pf[n++] = {rfd, POLLIN, 0};
    int r = poll(pf, n, static_cast<int>(std::min(left, 1.0) * 1000) + 1);
    if (r < 0 && errno != EINTR)
      Fail(std::string("poll failed: ") + std::strerror(errno));
  }
}

// ---------------------------------------------------------------------------

Comm::Comm(TcpMesh* mesh, std::vector<int> ranks)
    : mesh_(mesh), ranks_(std::move(ranks)) {
  rank_ = -1;
  for (size_t i = 0; i < ranks_.size(); ++i)
    if (ranks_[i] == mesh_->rank()) rank_ = static_cast<int>(i);
}

void Comm::SendRecv(int send_peer, const void* sbuf, size_t slen,
                    int recv_peer, void* rbuf, size_t rlen) {
  mesh_->SendRecv(send_peer >= 0 ? g(send_peer) : -1, sbuf, slen,
                  recv_peer >= 0 ? g(recv_peer) : -1, rbuf, rlen);
}

void Comm::Barrier() {
  uint64_t w = ~0ull;
  AllreduceBits(&w, 1, true);
}

void Comm::Bcast(void* buf, size_t len, int root) {
  int n = size();
  if (n <= 1 || len == 0) return;
  // Binomial tree rooted at `root` (relative rank vr = (rank - root) mod n).
  int vr = (rank_ - root + n) % n;
  int mask = 1;
  while (mask < n) {
    if (vr & mask) {
      int src = (vr - mask + root) % n;
      mesh_->Recv(g(src), buf, len);
      break;
    }
    mask <<= 1;
  }
  mask >>= 1;
  while (mask > 0) {
    if (vr + mask < n) {
      int dst = (vr + mask + root) % n;
      mesh_->Send(g(dst), buf, len);
    }
    mask >>= 1;
  }
}

void Comm::BcastBlob(std::string* blob, int root) {
  int64_t len = static_cast<int64_t>(blob->size());
  Bcast(&len, sizeof(len), root);
  if (rank_ != root) blob->resize(static_cast<size_t>(len));
  if (len > 0) Bcast(&(*blob)[0], static_cast<size_t>(len), root);
}

void Comm::GatherBlobs(const std::string& mine, int root,
                       std::vector<std::string>* out) {
  int n = size();
  if (rank_ == root) {
    out->assign(n, std::string());
    (*out)[root] = mine;
    for (int r = 0; r < n; ++r) {
      if (r == root) continue;
      int64_t len = 0;
      mesh_->Recv(g(r), &len, sizeof(len));
      (*out)[r].resize(static_cast<size_t>(len));
      if (len > 0) mesh_->Recv(g(r), &(*out)[r][0], static_cast<size_t>(len));
    }
  } else {
    int64_t len = static_cast<int64_t>(mine.size());
    mesh_->Send(g(root), &len, sizeof(len));
    if (len > 0) mesh_->Send(g(root), mine.data(), mine.size());
  }
}

void Comm::AllreduceBits(uint64_t* words, size_t n, bool bitwise_and) {
  int sz = size();
  if (sz <= 1 || n == 0) return;
  size_t bytes = n * sizeof(uint64_t);
  std::vector<uint64_t> tmp(n);
  if ((sz & (sz - 1)) == 0) {
    // Recursive doubling: log2(size) exchanges, no root bottleneck.
    for (int mask = 1; mask < sz; mask <<= 1) {
      int peer = rank_ ^ mask;
      mesh_->SendRecv(g(peer), words, bytes, g(peer), tmp.data(), bytes);
      if (bitwise_and)
        for (size_t i = 0; i < n; ++i) words[i] &= tmp[i];
      else
        for (size_t i = 0; i < n; ++i) words[i] |= tmp[i];
    }
    return;
  }
  if (rank_ == 0) {
    for (int r = 1; r < sz; ++r) {
      mesh_->Recv(g(r), tmp.data(), bytes);
      if (bitwise_and)
        for (size_t i = 0; i < n; ++i) words[i] &= tmp[i];
      else
        for (size_t i = 0; i < n; ++i) words[i] |= tmp[i];
    }
  } else {
    mesh_->Send(g(0), words, bytes);
  }
  Bcast(words, bytes, 0);
}

void Comm::Allgather(const void* send, size_t len, void* recv) {
  std::vector<int64_t> lens(size(), static_cast<int64_t>(len));
  Allgatherv(send, lens, recv);
}

void Comm::Allgatherv(const void* send, const std::vector<int64_t>& lens,
                      void* recv) {
  int n = size();
  std::vector<int64_t> offs(n + 1, 0);
  for (int i = 0; i < n; ++i) offs[i + 1] = offs[i] + lens[i];
  char* out = static_cast<char*>(recv);
  if (lens[rank_] > 0 && out + offs[rank_] != send)
    std::memcpy(out + offs[rank_], send, static_cast<size_t>(lens[rank_]));
  if (n <= 1) return;
  int64_t largest = 0;
  for (auto l : lens) largest = std::max(largest, l);
  if (largest <= 4096) {
    // Small blocks (split tables, handles): every rank hands its block to
    // every peer directly, so no block waits for a neighbour to forward it.
    for (int s = 1; s < n; ++s) {
      const int to = (rank_ + s) % n, from = (rank_ - s + n) % n;
      mesh_->SendRecv(g(to), out + offs[rank_], static_cast<size_t>(lens[rank_]),
                      g(from), out + offs[from], static_cast<size_t>(lens[from]));
    }
    return;
  }
  int right = (rank_ + 1) % n, left = (rank_ - 1 + n) % n;
  for (int s = 0; s < n - 1; ++s) {
    int sb = (rank_ - s + n) % n;      // block forwarded this step
    int rb = (rank_ - s - 1 + n) % n;  // block arriving this step
    mesh_->SendRecv(g(right), out + offs[sb], static_cast<size_t>(lens[sb]),
                    g(left), out + offs[rb], static_cast<size_t>(lens[rb]));
  }
}

void Comm::Alltoallv(const void* send, const std::vector<int64_t>& send_lens,
                     void* recv, const std::vector<int64_t>& recv_lens) {
  int n = size();
  std::vector<int64_t> so(n + 1, 0), ro(n + 1, 0);
  for (int i = 0; i < n; ++i) {
    so[i + 1] = so[i] + send_lens[i];
    ro[i + 1] = ro[i] + recv_lens[i];
  }
  const char* in = static_cast<const char*>(send);
  char* out = static_cast<char*>(recv);
  if (send_lens[rank_] != recv_lens[rank_])
    Fail("alltoall: self block size mismatch");
  if (send_lens[rank_] > 0)
    std::memcpy(out + ro[rank_], in + so[rank_],
                static_cast<size_t>(send_lens[rank_]));
  for (int s = 1; s < n; ++s) {
    int to = (rank_ + s) % n, from = (rank_ - s + n) % n;
    mesh_->SendRecv(g(to), in + so[to], static_cast<size_t>(send_lens[to]),
                    g(from), out + ro[from],
                    static_cast<size_t>(recv_lens[from]));
  }
}

void Comm::Allreduce(void* buf, int64_t count, DataType dtype, ReduceOp op) {
  int n = size();
  if (n <= 1 || count == 0) return;
  size_t es = DataTypeSize(dtype);
  char* data = static_cast<char*>(buf);
  int64_t bytes = count * static_cast<int64_t>(es);
  if (bytes < 32768 || count < n) {
    // Latency path: recursive doubling when size is a power of two,
    // otherwise reduce at rank 0 and broadcast.
    std::vector<char> tmp(static_cast<size_t>(bytes));
    if ((n & (n - 1)) == 0) {
      for (int mask = 1; mask < n; mask <<= 1) {
        int peer = rank_ ^ mask;
        mesh_->SendRecv(g(peer), data, bytes, g(peer), tmp.data(), bytes);
        // Keep operand order identical on both sides so that every rank
        // computes bit-identical floating point results.
        if (rank_ < peer) {
          ReduceInto(data, tmp.data(), count, dtype, op);
        } else {
          ReduceInto(tmp.data(), data, count, dtype, op);
          std::memcpy(data, tmp.data(), static_cast<size_t>(bytes));
        }
      }
    } else {
      if (rank_ == 0) {
        for (int r = 1; r < n; ++r) {
          mesh_->Recv(g(r), tmp.data(), bytes);
          ReduceInto(data, tmp.data(), count, dtype, op);
        }
      } else {
        mesh_->Send(g(0), data, bytes);
      }
      Bcast(data, bytes, 0);
    }
    return;
  }
  // Bandwidth path: ring reduce-scatter followed by ring allgather.
  std::vector<int64_t> start(n + 1);
  for (int i = 0; i <= n; ++i) start[i] = count * i / n;
  int64_t max_chunk = 0;
  for (int i = 0; i < n; ++i)
    max_chunk = std::max(max_chunk, start[i + 1] - start[i]);
  std::vector<char> tmp(static_cast<size_t>(max_chunk) * es);
  int right = (rank_ + 1) % n, left = (rank_ - 1 + n) % n;
  for (int s = 0; s < n - 1; ++s) {
    int sc = (rank_ - s + n) % n;
    int rc = (rank_ - s - 1 + n) % n;
    int64_t sn = start[sc + 1] - start[sc], rn = start[rc + 1] - start[rc];
    mesh_->SendRecv(g(right), data + start[sc] * es, sn * es, g(left),
                    tmp.data(), rn * es);
    ReduceInto(data + start[rc] * es, tmp.data(), rn, dtype, op);
  }
  // Rank r now owns the fully reduced chunk (r + 1) mod n.
  for (int s = 0; s < n - 1; ++s) {
    int sc = (rank_ + 1 - s + n) % n;
    int rc = (rank_ - s + n) % n;
    int64_t sn = start[sc + 1] - start[sc], rn = start[rc + 1] - start[rc];
    mesh_->SendRecv(g(right), data + start[sc] * es, sn * es, g(left),
                    data + start[rc] * es, rn * es);
  }
}

// ---------------------------------------------------------------------------
// CPU reduction / scale kernels

namespace {

template <typename T>
void ReduceTyped(T* d, const T* s, int64_t n, ReduceOp op) {
  switch (op) {
  case ReduceOp::MIN:
    for (int64_t i = 0; i < n; ++i) d[i] = s[i] < d[i] ? s[i] : d[i];
    break;
  case ReduceOp::MAX:
    for (int64_t i = 0; i < n; ++i) d[i] = s[i] > d[i] ? s[i] : d[i];
    break;
  case ReduceOp::PRODUCT:
    for (int64_t i = 0; i < n; ++i) d[i] = static_cast<T>(d[i] * s[i]);
    break;
  default:
    for (int64_t i = 0; i < n; ++i) d[i] = static_cast<T>(d[i] + s[i]);
  }
}

inline float Combine(float a, float b, ReduceOp op) {
  switch (op) {
  case ReduceOp::MIN: return b < a ? b : a;
  case ReduceOp::MAX: return b > a ? b : a;
  case ReduceOp::PRODUCT: return a * b;
  default: return a + b;
  }
}

void ReduceHalf(uint16_t* d, const uint16_t* s, int64_t n, ReduceOp op) {
  if (op == ReduceOp::SUM || op == ReduceOp::AVERAGE || op == ReduceOp::ADASUM) {
    HalfSum(d, s, n);  // AVX2 + F16C when the CPU has them
    return;
  }
  for (int64_t i = 0; i < n; ++i)
    d[i] = FloatToHalfBits(
        Combine(HalfBitsToFloat(d[i]), HalfBitsToFloat(s[i]), op));
}

void ReduceBF16(uint16_t* d, const uint16_t* s, int64_t n, ReduceOp op) {
  if (op == ReduceOp::SUM || op == ReduceOp::AVERAGE || op == ReduceOp::ADASUM) {
    BF16Sum(d, s, n);
    return;
  }
  for (int64_t i = 0; i < n; ++i)
    d[i] = FloatToBF16Bits(
        Combine(BF16BitsToFloat(d[i]), BF16BitsToFloat(s[i]), op));
}

void ReduceBool(uint8_t* d, const uint8_t* s, int64_t n, ReduceOp op) {
  // Sum/max act as logical OR, product/min as logical AND.
  bool is_and = (op == ReduceOp::MIN || op == ReduceOp::PRODUCT);
  for (int64_t i = 0; i < n; ++i)
    d[i] = is_and ? ((d[i] != 0) && (s[i] != 0)) : ((d[i] != 0) || (s[i] != 0));
}

template <typename T> void ScaleTyped(T* p, int64_t n, double f) {
  for (int64_t i = 0; i < n; ++i) p[i] = static_cast<T>(p[i] * f);
}

}  // namespace

}  // namespace hvd

namespace hvd {

void ReduceInto(void* dst, const void* src, int64_t count, DataType dtype,
                ReduceOp op) {
  switch (dtype) {
  case DataType::UINT8:
    ReduceTyped(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), count, op);
    break;
  case DataType::INT8:
    ReduceTyped(static_cast<int8_t*>(dst), static_cast<const int8_t*>(src), count, op);
    break;
  case DataType::UINT16:
    ReduceTyped(static_cast<uint16_t*>(dst), static_cast<const uint16_t*>(src), count, op);
    break;
  case DataType::INT16:
    ReduceTyped(static_cast<int16_t*>(dst), static_cast<const int16_t*>(src), count, op);
    break;
  case DataType::INT32:
    ReduceTyped(static_cast<int32_t*>(dst), static_cast<const int32_t*>(src), count, op);
    break;
  case DataType::INT64:
    ReduceTyped(static_cast<int64_t*>(dst), static_cast<const int64_t*>(src), count, op);
    break;
  case DataType::FLOAT32:
    ReduceTyped(static_cast<float*>(dst), static_cast<const float*>(src), count, op);
    break;
  case DataType::FLOAT64:
    ReduceTyped(static_cast<double*>(dst), static_cast<const double*>(src), count, op);
    break;
  case DataType::FLOAT16:
    ReduceHalf(static_cast<uint16_t*>(dst), static_cast<const uint16_t*>(src), count, op);
    break;
  case DataType::BFLOAT16:
    ReduceBF16(static_cast<uint16_t*>(dst), static_cast<const uint16_t*>(src), count, op);
    break;
  case DataType::BOOL:
    ReduceBool(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), count, op);
    break;
  }
}

void ScaleBufferCPU(void* buf, int64_t count, DataType dtype, double factor) {
  if (factor == 1.0) return;
  switch (dtype) {
  case DataType::UINT8: ScaleTyped(static_cast<uint8_t*>(buf), count, factor); break;
  case DataType::INT8: ScaleTyped(static_cast<int8_t*>(buf), count, factor); break;
  case DataType::UINT16: ScaleTyped(static_cast<uint16_t*>(buf), count, factor); break;
  case DataType::INT16: ScaleTyped(static_cast<int16_t*>(buf), count, factor); break;
  case DataType::INT32: ScaleTyped(static_cast<int32_t*>(buf), count, factor); break;
  case DataType::INT64: ScaleTyped(static_cast<int64_t*>(buf), count, factor); break;
  case DataType::FLOAT32: {
    float* p = static_cast<float*>(buf);
    float f = static_cast<float>(factor);
    for (int64_t i = 0; i < count; ++i) p[i] *= f;
    break;
  }
  case DataType::FLOAT64: ScaleTyped(static_cast<double*>(buf), count, factor); break;
  case DataType::FLOAT16:
    HalfScale(static_cast<uint16_t*>(buf), count, static_cast<float>(factor));
    break;
  case DataType::BFLOAT16:
    BF16Scale(static_cast<uint16_t*>(buf), count, static_cast<float>(factor));
    break;
  case DataType::BOOL: break;
  }
}

}  // namespace hvd
