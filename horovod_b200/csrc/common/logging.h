// Leveled logging to stderr: HVD_LOG(WARNING) << "...";
// Level from HOROVOD_LOG_LEVEL (trace|debug|info|warning|error|fatal, default
// warning); HOROVOD_LOG_HIDE_TIME drops the timestamp.
//
// Parity: horovod/common/logging.h:38-56, logging.cc:55-92.
#pragma once

#include <sstream>
#include <string>

namespace hvd {

enum class LogLevel { TRACE = 0, DEBUG, INFO, WARNING, ERROR, FATAL };

LogLevel MinLogLevel();
void ResetLogLevelFromEnv();
// Rank shown in the prefix of every message (-1 = unknown yet).
void SetLogRank(int rank);

class LogMessage : public std::ostringstream {
public:
  LogMessage(const char* file, int line, LogLevel level, int rank = -2);
  ~LogMessage() override;

private:
  const char* file_;
  int line_;
  LogLevel level_;
  int rank_;
};

}  // namespace hvd

#define HVD_LOG_ENABLED(lvl) (::hvd::LogLevel::lvl >= ::hvd::MinLogLevel())
#define HVD_LOG(lvl)                                                          \
  if (HVD_LOG_ENABLED(lvl))                                                   \
  ::hvd::LogMessage(__FILE__, __LINE__, ::hvd::LogLevel::lvl)
#define HVD_LOG_RANK(lvl, rank)                                               \
  if (HVD_LOG_ENABLED(lvl))                                                   \
  ::hvd::LogMessage(__FILE__, __LINE__, ::hvd::LogLevel::lvl, rank)
