// Key-value stores used to bootstrap the TCP mesh.
//
// HttpStore talks to the launcher's rendezvous server: PUT /scope/key stores
// a value, GET /scope/key returns it (404 until it exists), DELETE
// /scope/key tells the server this rank is done with the scope.
// MemoryStore serves single-process jobs and pre-resolved address lists.
//
// Parity: horovod/common/gloo/http_store.cc:33-135 and memory_store.cc:27-64.
#pragma once

#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace hvd {

class Store {
public:
  virtual ~Store() = default;
  virtual void Set(const std::string& key, const std::string& value) = 0;
  // Blocks (polling) until the key exists or timeout_s elapses; throws
  // TransportError on timeout.
  virtual std::string Get(const std::string& key, double timeout_s) = 0;
  virtual void Finalize() {}
};

class MemoryStore : public Store {
public:
  void Set(const std::string& key, const std::string& value) override;
  std::string Get(const std::string& key, double timeout_s) override;

private:
  std::mutex mu_;
  std::map<std::string, std::string> kv_;
};

class HttpStore : public Store {
public:
  HttpStore(std::string host, int port, std::string scope, int rank)
      : host_(std::move(host)), port_(port), scope_(std::move(scope)),
        rank_(rank) {}
  void Set(const std::string& key, const std::string& value) override;
  std::string Get(const std::string& key, double timeout_s) override;
  // DELETE /scope/<rank>: lets the server drop the scope once all ranks left.
  void Finalize() override;

  // One HTTP exchange. Returns the status code; body receives the payload.
  static int Request(const std::string& host, int port,
                     const std::string& method, const std::string& path,
                     const std::string& payload, std::string* body,
                     double timeout_s);

private:
  std::string host_;
  int port_;
  std::string scope_;
  int rank_;
};

}  // namespace hvd
