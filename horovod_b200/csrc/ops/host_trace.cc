#include "host_trace.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace hvd {
namespace host_trace {

namespace {
struct Sum {
  double us = 0;
  long n = 0;
};
std::mutex g_mu;
std::map<int, std::vector<std::pair<std::string, Sum>>> g_sums;  // marks in first-seen order
thread_local int t_type = -1;
thread_local std::chrono::steady_clock::time_point t_last;
}  // namespace

bool Enabled() {
  static const bool on = [] {
    const char* v = std::getenv("HOROVOD_HOST_TRACE");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return on;
}

void Begin(int type) {
  if (!Enabled()) return;
  t_type = type;
  t_last = std::chrono::steady_clock::now();
}

void Mark(const char* label) {
  if (!Enabled() || t_type < 0) return;
  const auto now = std::chrono::steady_clock::now();
  const double us = std::chrono::duration<double, std::micro>(now - t_last).count();
  t_last = now;
  std::lock_guard<std::mutex> l(g_mu);
  auto& marks = g_sums[t_type];
  for (auto& m : marks) {
    if (m.first == label) {
      m.second.us += us;
      ++m.second.n;
      return;
    }
  }
  marks.push_back({label, Sum{us, 1}});
}

void Report(int rank) {
  if (!Enabled()) return;
  std::lock_guard<std::mutex> l(g_mu);
  for (auto& kv : g_sums) {
    std::string line = "[host trace] rank " + std::to_string(rank) + " response type " +
                       std::to_string(kv.first) + ":";
    for (auto& m : kv.second) {
      char buf[128];
      std::snprintf(buf, sizeof(buf), " %s %.2f us x%ld;", m.first.c_str(),
                    m.second.us / static_cast<double>(m.second.n), m.second.n);
      line += buf;
    }
    std::fprintf(stderr, "%s\n", line.c_str());
  }
  g_sums.clear();
}

}  // namespace host_trace
}  // namespace hvd
