#include "store.h"

#include <algorithm>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <thread>

#include <netdb.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include "mesh.h"

namespace hvd {

namespace {
using Clock = std::chrono::steady_clock;
double Since(Clock::time_point t0) {
  return std::chrono::duration<double>(Clock::now() - t0).count();
}
}  // namespace

void MemoryStore::Set(const std::string& key, const std::string& value) {
  std::lock_guard<std::mutex> l(mu_);
  kv_[key] = value;
}

std::string MemoryStore::Get(const std::string& key, double timeout_s) {
  auto t0 = Clock::now();
  for (;;) {
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = kv_.find(key);
      if (it != kv_.end()) return it->second;
    }
    if (Since(t0) > timeout_s)
      throw TransportError("hvd store: key '" + key + "' never appeared");
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

int HttpStore::Request(const std::string& host, int port,
                       const std::string& method, const std::string& path,
                       const std::string& payload, std::string* body,
                       double timeout_s) {
  struct addrinfo hints;
  std::memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  struct addrinfo* res = nullptr;
  if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0)
    return -1;
  int fd = -1;
  for (auto* ai = res; ai != nullptr; ai = ai->ai_next) {
    fd = socket(ai->ai_family, ai->ai_socktype, ai->ai_protocol);
    if (fd < 0) continue;
    if (connect(fd, ai->ai_addr, ai->ai_addrlen) == 0) break;
    close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) return -1;
  std::string req = method + " " + path + " HTTP/1.0\r\nHost: " + host +
                    "\r\nContent-Length: " + std::to_string(payload.size()) +
                    "\r\nConnection: close\r\n\r\n" + payload;
  size_t off = 0;
  while (off < req.size()) {
    ssize_t n = ::send(fd, req.data() + off, req.size() - off, MSG_NOSIGNAL);
    if (n < 0) {
      if (errno == EINTR) continue;
      close(fd);
      return -1;
    }
    off += static_cast<size_t>(n);
  }
  std::string resp;
  auto t0 = Clock::now();
  char buf[4096];
  for (;;) {
    double left = timeout_s - Since(t0);
    if (left <= 0) {
      close(fd);
      return -1;
    }
    struct pollfd pf = {fd, POLLIN, 0};
    int r = poll(&pf, 1, static_cast<int>(std::min(left, 1.0) * 1000) + 1);
    if (r < 0 && errno != EINTR) break;
    if (r <= 0) continue;
    ssize_t n = ::recv(fd, buf, sizeof(buf), 0);
    if (n == 0) break;
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      break;
    }
    resp.append(buf, static_cast<size_t>(n));
  }
  close(fd);
  // "HTTP/1.x NNN ..."
  auto sp = resp.find(' ');
  if (sp == std::string::npos || sp + 4 > resp.size()) return -1;
  int code = std::atoi(resp.c_str() + sp + 1);
  auto hdr_end = resp.find("\r\n\r\n");
  if (body != nullptr)
    *body = hdr_end == std::string::npos ? std::string() : resp.substr(hdr_end + 4);
  return code;
}

void HttpStore::Set(const std::string& key, const std::string& value) {
  auto t0 = Clock::now();
  int backoff_ms = 10;
  for (;;) {
    int code = Request(host_, port_, "PUT", "/" + scope_ + "/" + key, value,
                       nullptr, 30.0);
    if (code == 200) return;
    if (Since(t0) > 60.0)
      throw TransportError("hvd store: PUT " + scope_ + "/" + key +
                           " failed (HTTP " + std::to_string(code) + ")");
    std::this_thread::sleep_for(std::chrono::milliseconds(backoff_ms));
    backoff_ms = std::min(backoff_ms * 2, 500);
  }
}

std::string HttpStore::Get(const std::string& key, double timeout_s) {
  auto t0 = Clock::now();
  for (;;) {
    std::string body;
    // Some scopes block on the server side (elastic barrier), so the single
    // request gets the whole remaining budget.
    double left = std::max(1.0, timeout_s - Since(t0));
    int code = Request(host_, port_, "GET", "/" + scope_ + "/" + key, "",
                       &body, left);
    if (code == 200) return body;
    if (Since(t0) > timeout_s)
      throw TransportError("hvd store: GET " + scope_ + "/" + key +
                           " timed out (last HTTP status " +
                           std::to_string(code) + ")");
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
  }
}

void HttpStore::Finalize() {
  Request(host_, port_, "DELETE", "/" + scope_ + "/" + std::to_string(rank_),
          "", nullptr, 5.0);
}

}  // namespace hvd
