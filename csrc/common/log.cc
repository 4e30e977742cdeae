#include "log.h"

#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "clock.h"
#include "env.h"

namespace pccl {

static std::mutex g_log_mu;
static const char* kNames[] = {"TRACE", "DEBUG", "INFO", "WARN", "ERROR", "CRITICAL", "OFF"};

LogLevel Logger::parseLevel(const std::string& s, LogLevel dflt) {
  std::string u = s;
  std::transform(u.begin(), u.end(), u.begin(), ::toupper);
  for (int i = 0; i < 7; ++i)
    if (u == kNames[i]) return static_cast<LogLevel>(i);
  return dflt;
}

static void mkdirs(const std::string& dir) {
  std::string cur;
  for (size_t i = 0; i <= dir.size(); ++i) {
    if (i == dir.size() || dir[i] == '/') {
      if (!cur.empty()) ::mkdir(cur.c_str(), 0777);
    }
    if (i < dir.size()) cur.push_back(dir[i]);
  }
}

Logger::Logger() : file_(nullptr) {
  std::memset(counts_, 0, sizeof(counts_));
  level_ = parseLevel(LaunchEnvironments::getEnv("PCCL_LOG_LEVEL"), LogLevel::Warn);
  to_terminal_ = LaunchEnvironments::getBool("PCCL_LOG_TO_TERMINAL", false);
  std::string dir = LaunchEnvironments::getStr("PCCL_LOG_DIR", "/tmp/pccl/log");
  std::string name = LaunchEnvironments::getStr(
      "PCCL_LOG_FILENAME", launchTimestamp() + "." + std::to_string(::getpid()) + ".log");
  mkdirs(dir);
  path_ = dir + "/" + name;
  file_ = std::fopen(path_.c_str(), "w");   // truncating sink, like the reference
}

Logger::~Logger() {
  if (file_) std::fclose(static_cast<FILE*>(file_));
}

Logger& Logger::get() {
  static Logger l;
  return l;
}

uint64_t Logger::count(LogLevel lvl) const { return counts_[static_cast<int>(lvl)]; }

void Logger::log(LogLevel lvl, const char* file, int line, const char* fmt, ...) {
  char msg[2048];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  const char* base = std::strrchr(file, '/');
  base = base ? base + 1 : file;
  std::string ts = nowString();
  std::lock_guard<std::mutex> g(g_log_mu);
  counts_[static_cast<int>(lvl)]++;
  FILE* f = static_cast<FILE*>(file_);
  if (f) {
    std::fprintf(f, "[%s] [pccl] [%s] [%s:%d] %s\n", ts.c_str(), kNames[static_cast<int>(lvl)], base, line, msg);
    if (lvl >= level_) std::fflush(f);
  }
  if (to_terminal_)
    std::fprintf(stderr, "[%s] [pccl] [%s] [%s:%d] %s\n", ts.c_str(), kNames[static_cast<int>(lvl)], base, line, msg);
}

}  // namespace pccl
