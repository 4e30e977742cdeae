// Logger "pccl": file sink plus optional stderr sink, level chosen by PCCL_LOG_LEVEL.
//
// Same environment contract as the reference logger (csrc/common/logging.cc:30-62,
// include/common/logging.h:12-33): PCCL_LOG_LEVEL in TRACE..CRITICAL (default WARN),
// PCCL_LOG_TO_TERMINAL, PCCL_LOG_FILENAME (default "<launch time>.log"), debug-only macros that
// vanish unless PCCL_DEBUG is defined.  Differences: no spdlog (printf-style, one mutex), the log
// directory is created if missing (the reference never creates /tmp/pccl/log), and counters of
// messages per level are kept for Engine.stats().
#pragma once
#include <cstdarg>
#include <cstdint>
#include <string>

namespace pccl {

enum class LogLevel : int { Trace = 0, Debug, Info, Warn, Error, Critical, Off };

class Logger {
 public:
  static Logger& get();
  void log(LogLevel lvl, const char* file, int line, const char* fmt, ...)
      __attribute__((format(printf, 5, 6)));
  bool enabled(LogLevel lvl) const { return static_cast<int>(lvl) >= static_cast<int>(level_); }
  LogLevel level() const { return level_; }
  void setLevel(LogLevel l) { level_ = l; }
  const std::string& path() const { return path_; }
  uint64_t count(LogLevel lvl) const;
  static LogLevel parseLevel(const std::string& s, LogLevel dflt);

 private:
  Logger();
  ~Logger();
  LogLevel level_;
  bool to_terminal_;
  std::string path_;
  void* file_;   // FILE*
  uint64_t counts_[7];
};

}  // namespace pccl

#define PCCL_LOG_AT(lvl, ...)                                                        \
  do {                                                                               \
    if (::pccl::Logger::get().enabled(lvl))                                          \
      ::pccl::Logger::get().log(lvl, __FILE__, __LINE__, __VA_ARGS__);               \
  } while (0)
#define PCCL_LOG_TRACE(...) PCCL_LOG_AT(::pccl::LogLevel::Trace, __VA_ARGS__)
#define PCCL_LOG_DEBUG(...) PCCL_LOG_AT(::pccl::LogLevel::Debug, __VA_ARGS__)
#define PCCL_LOG_INFO(...) PCCL_LOG_AT(::pccl::LogLevel::Info, __VA_ARGS__)
#define PCCL_LOG_WARN(...) PCCL_LOG_AT(::pccl::LogLevel::Warn, __VA_ARGS__)
#define PCCL_LOG_ERROR(...) PCCL_LOG_AT(::pccl::LogLevel::Error, __VA_ARGS__)
#define PCCL_LOG_CRITICAL(...) PCCL_LOG_AT(::pccl::LogLevel::Critical, __VA_ARGS__)
#ifdef PCCL_DEBUG
#define PCCL_DLOG_TRACE(...) PCCL_LOG_TRACE(__VA_ARGS__)
#define PCCL_DLOG_DEBUG(...) PCCL_LOG_DEBUG(__VA_ARGS__)
#define PCCL_DLOG_INFO(...) PCCL_LOG_INFO(__VA_ARGS__)
#else
#define PCCL_DLOG_TRACE(...) ((void)0)
#define PCCL_DLOG_DEBUG(...) ((void)0)
#define PCCL_DLOG_INFO(...) ((void)0)
#endif
