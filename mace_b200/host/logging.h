// Env-gated logging of the host layer with the names and switches of MACE's logger:
//   LOG(INFO | WARNING | ERROR)   shown when the level passes MACE_CPP_MIN_LOG_LEVEL
//                                 (I / W / E / F or the full word; default: everything)
//   VLOG(n)                       an INFO line shown when n <= MACE_CPP_MIN_VLOG_LEVEL (default 0)
//   MACE_LATENCY_LOGGER(n, ...)   "<message> started" / "<message> latency: <us> us" at VLOG(n)
//   EnvConfEnabled(name)          an environment switch: set, not empty and not starting with '0'
// (include/mace/port/logger.h:24-70, mace/port/logger.cc:33-80, include/mace/utils/logging.h:
// 34-124, mace/utils/conf_util.h:26-29).  A line is "<I|W|E|F> <file>:<line>] <message>" and goes
// to stderr, or to the sink a test or an embedding application installs.  Both environment
// variables are read once, at the first message; SetVLogLevelForTest overrides the second.
// LOG(FATAL) is not offered: the host layer reports errors through MaceStatus.
#ifndef MACE_B200_HOST_LOGGING_H_
#define MACE_B200_HOST_LOGGING_H_

#include <atomic>
#include <cctype>
#include <chrono>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <string>

namespace mace {

enum LogLevel { INVALID_MIN = 0, INFO = 1, WARNING = 2, ERROR = 3, FATAL = 4, INVALID_MAX };

typedef void (*LogSink)(int severity, const char *line);

namespace logging_internal {

inline std::atomic<LogSink> &Sink() {
  static std::atomic<LogSink> sink{nullptr};
  return sink;
}

inline std::atomic<int> &VLogOverride() {
  static std::atomic<int> level{INT_MIN};
  return level;
}

inline LogLevel LogLevelFromStr(const char *s) {
  if (s == nullptr) return INVALID_MIN;
  std::string u(s);
  for (auto &c : u) c = static_cast<char>(std::toupper(static_cast<unsigned char>(c)));
  if (u == "I" || u == "INFO") return INFO;
  if (u == "W" || u == "WARNING") return WARNING;
  if (u == "E" || u == "ERROR") return ERROR;
  if (u == "F" || u == "FATAL") return FATAL;
  return INVALID_MIN;
}

inline LogLevel MinLogLevelFromEnv() {
  static const LogLevel level = LogLevelFromStr(std::getenv("MACE_CPP_MIN_LOG_LEVEL"));
  return level;
}

inline int MinVLogLevelFromEnv() {
  static const int level = [] {
    const char *s = std::getenv("MACE_CPP_MIN_VLOG_LEVEL");
    return s != nullptr ? std::atoi(s) : 0;
  }();
  return level;
}

}  // namespace logging_internal

inline void SetLogSink(LogSink sink) { logging_internal::Sink().store(sink); }
// level = INT_MIN returns to the environment's value.
inline void SetVLogLevelForTest(int level) { logging_internal::VLogOverride().store(level); }

inline bool ShouldGenerateVLogMessage(int vlog_level) {
  const int forced = logging_internal::VLogOverride().load();
  const int limit = forced != INT_MIN ? forced : logging_internal::MinVLogLevelFromEnv();
  return logging_internal::MinLogLevelFromEnv() <= INFO && vlog_level <= limit;
}

inline bool EnvConfEnabled(const char *name) {
  const char *env = std::getenv(name);
  return !(env == nullptr || env[0] == 0 || env[0] == '0');
}

class Logger : public std::ostringstream {
 public:
  Logger(const char *fname, int line, LogLevel severity) : fname_(fname), line_(line), severity_(severity) {}
  ~Logger() override {
    if (severity_ < logging_internal::MinLogLevelFromEnv()) return;
    const char *base = std::strrchr(fname_, '/');
    std::ostringstream out;
    out << "IWEF"[(severity_ >= INFO && severity_ <= FATAL ? severity_ : INFO) - 1] << ' '
        << (base != nullptr ? base + 1 : fname_) << ':' << line_ << "] " << str();
    const LogSink sink = logging_internal::Sink().load();
    if (sink != nullptr) {
      sink(static_cast<int>(severity_), out.str().c_str());
    } else {
      std::fprintf(stderr, "%s\n", out.str().c_str());
    }
  }

 private:
  const char *fname_;
  int line_;
  LogLevel severity_;
};

class LatencyLogger {
 public:
  LatencyLogger(int vlog_level, const std::string &message) : vlog_level_(vlog_level), message_(message) {
    if (ShouldGenerateVLogMessage(vlog_level_)) {
      start_ = std::chrono::steady_clock::now();
      Logger(__FILE__, __LINE__, INFO) << message_ << " started";
    }
  }
  ~LatencyLogger() {
    if (ShouldGenerateVLogMessage(vlog_level_)) {
      const auto us = std::chrono::duration_cast<std::chrono::microseconds>(
                          std::chrono::steady_clock::now() - start_).count();
      Logger(__FILE__, __LINE__, INFO) << message_ << " latency: " << us << " us";
    }
  }

 private:
  int vlog_level_;
  std::string message_;
  std::chrono::steady_clock::time_point start_;
};

}  // namespace mace

#define LOG(severity) ::mace::Logger(__FILE__, __LINE__, ::mace::severity)
#define VLOG_IS_ON(vll) (::mace::ShouldGenerateVLogMessage(vll))
#define VLOG(vll) \
  if (VLOG_IS_ON(vll)) LOG(INFO)
#define MACE_LATENCY_LOGGER(vlog_level, message) \
  ::mace::LatencyLogger mace_latency_logger_##__LINE__(vlog_level, VLOG_IS_ON(vlog_level) ? (message) : std::string())

#endif  // MACE_B200_HOST_LOGGING_H_
