#include "logging.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>

namespace hvd {

namespace {
std::atomic<int> g_level{-1};
std::atomic<int> g_rank{-1};
std::atomic<int> g_hide_time{-1};

LogLevel ParseLevel(const char* v) {
  if (v == nullptr) return LogLevel::WARNING;
  std::string s(v);
  std::transform(s.begin(), s.end(), s.begin(), ::tolower);
  if (s == "trace") return LogLevel::TRACE;
  if (s == "debug") return LogLevel::DEBUG;
  if (s == "info") return LogLevel::INFO;
  if (s == "warning" || s == "warn") return LogLevel::WARNING;
  if (s == "error") return LogLevel::ERROR;
  if (s == "fatal") return LogLevel::FATAL;
  return LogLevel::WARNING;
}
}  // namespace

void ResetLogLevelFromEnv() {
  g_level = static_cast<int>(ParseLevel(std::getenv("HOROVOD_LOG_LEVEL")));
  const char* h = std::getenv("HOROVOD_LOG_HIDE_TIME");
  g_hide_time = (h != nullptr && std::strtol(h, nullptr, 10) > 0) ? 1 : 0;
}

LogLevel MinLogLevel() {
  if (g_level.load(std::memory_order_relaxed) < 0) ResetLogLevelFromEnv();
  return static_cast<LogLevel>(g_level.load(std::memory_order_relaxed));
}

void SetLogRank(int rank) { g_rank = rank; }

LogMessage::LogMessage(const char* file, int line, LogLevel level, int rank)
    : file_(file), line_(line), level_(level),
      rank_(rank == -2 ? g_rank.load() : rank) {}

LogMessage::~LogMessage() {
  static const char* names[] = {"TRACE", "DEBUG", "INFO",
                                "WARNING", "ERROR", "FATAL"};
  const char* base = std::strrchr(file_, '/');
  base = base ? base + 1 : file_;
  char when[64] = "";
  if (g_hide_time.load() <= 0) {
    auto now = std::chrono::system_clock::now();
    std::time_t t = std::chrono::system_clock::to_time_t(now);
    int us = static_cast<int>(
        std::chrono::duration_cast<std::chrono::microseconds>(
            now.time_since_epoch()).count() % 1000000);
    std::tm tm_buf;
    localtime_r(&t, &tm_buf);
    char hms[32];
    std::strftime(hms, sizeof(hms), "%Y-%m-%d %H:%M:%S", &tm_buf);
    std::snprintf(when, sizeof(when), "%s.%06d: ", hms, us);
  }
  char rank[24] = "";
  if (rank_ >= 0) std::snprintf(rank, sizeof(rank), "[%d]", rank_);
  std::fprintf(stderr, "[%s%s %s:%d]%s %s\n", when,
               names[static_cast<int>(level_)], base, line_, rank,
               str().c_str());
  if (level_ == LogLevel::FATAL) std::abort();
}

}  // namespace hvd
