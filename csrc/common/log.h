// Leveled stderr logger for the native layer.
//
// Line format: "[MCCL LEVEL epoch_ms file:line] message", one line per call,
// serialised by a process-wide mutex.  The threshold is read once from
// MCCL_LOG_LEVEL (TRACE, DEBUG, INFO, WARN, ERROR, FATAL, OFF; default WARN).
// Behavioural parity: reference csrc/common/Logging.hpp:22-102.
#pragma once

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

namespace mccl {

enum class LogLevel : int { TRACE = 0, DEBUG, INFO, WARN, ERROR, FATAL, OFF };

inline LogLevel parse_log_level(const char* s) {
  if (!s || !*s) return LogLevel::WARN;
  std::string v(s);
  for (auto& c : v) c = static_cast<char>(::toupper(c));
  if (v == "TRACE") return LogLevel::TRACE;
  if (v == "DEBUG") return LogLevel::DEBUG;
  if (v == "INFO") return LogLevel::INFO;
  if (v == "WARN" || v == "WARNING") return LogLevel::WARN;
  if (v == "ERROR") return LogLevel::ERROR;
  if (v == "FATAL") return LogLevel::FATAL;
  if (v == "OFF" || v == "NONE") return LogLevel::OFF;
  return LogLevel::WARN;
}

inline LogLevel& log_threshold() {
  static LogLevel lvl = parse_log_level(std::getenv("MCCL_LOG_LEVEL"));
  return lvl;
}

inline std::mutex& log_mutex() {
  static std::mutex mu;
  return mu;
}

inline const char* level_name(LogLevel l) {
  switch (l) {
    case LogLevel::TRACE: return "TRACE";
    case LogLevel::DEBUG: return "DEBUG";
    case LogLevel::INFO: return "INFO";
    case LogLevel::WARN: return "WARN";
    case LogLevel::ERROR: return "ERROR";
    case LogLevel::FATAL: return "FATAL";
    default: return "OFF";
  }
}

inline bool log_enabled(LogLevel l) {
  return static_cast<int>(l) >= static_cast<int>(log_threshold()) &&
         log_threshold() != LogLevel::OFF;
}

#if defined(__GNUC__)
__attribute__((format(printf, 4, 5)))
#endif
inline void
logf(LogLevel lvl, const char* file, int line, const char* fmt, ...) {
  if (!log_enabled(lvl)) return;
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  const char* base = std::strrchr(file, '/');
  base = base ? base + 1 : file;
  auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(
                std::chrono::system_clock::now().time_since_epoch())
                .count();
  std::lock_guard<std::mutex> g(log_mutex());
  std::fprintf(stderr, "[MCCL %s %lld %s:%d] %s\n", level_name(lvl),
               static_cast<long long>(ms), base, line, buf);
  std::fflush(stderr);
}

}  // namespace mccl

#define MCCL_TRACE(...) ::mccl::logf(::mccl::LogLevel::TRACE, __FILE__, __LINE__, __VA_ARGS__)
#define MCCL_DEBUG(...) ::mccl::logf(::mccl::LogLevel::DEBUG, __FILE__, __LINE__, __VA_ARGS__)
#define MCCL_INFO(...) ::mccl::logf(::mccl::LogLevel::INFO, __FILE__, __LINE__, __VA_ARGS__)
#define MCCL_WARN(...) ::mccl::logf(::mccl::LogLevel::WARN, __FILE__, __LINE__, __VA_ARGS__)
#define MCCL_ERROR(...) ::mccl::logf(::mccl::LogLevel::ERROR, __FILE__, __LINE__, __VA_ARGS__)
#define MCCL_FATAL(...) ::mccl::logf(::mccl::LogLevel::FATAL, __FILE__, __LINE__, __VA_ARGS__)
// Unrecoverable invariant violation: log and terminate the process.
#define MCCL_ABORT(...)            \
  do {                             \
    MCCL_FATAL(__VA_ARGS__);       \
    std::terminate();              \
  } while (0)
