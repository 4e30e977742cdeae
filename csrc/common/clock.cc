#include "clock.h"

#include <chrono>
#include <cstdio>
#include <ctime>

namespace pccl {

static std::string stamp(const char* fmt_date, bool with_date) {
  using namespace std::chrono;
  auto now = system_clock::now();
  auto us = duration_cast<microseconds>(now.time_since_epoch()).count() % 1000000;
  std::time_t t = system_clock::to_time_t(now);
  std::tm tm{};
  localtime_r(&t, &tm);
  char buf[64], out[96];
  std::strftime(buf, sizeof(buf), fmt_date, &tm);
  std::snprintf(out, sizeof(out), "%s.%06lld", buf, static_cast<long long>(us));
  (void)with_date;
  return out;
}

const std::string& launchTimestamp() {
  static const std::string s = stamp("%H-%M-%S", false);
  return s;
}

namespace { struct Init { Init() { (void)launchTimestamp(); } } init_at_load; }

uint64_t nowNanos() {
  using namespace std::chrono;
  return duration_cast<nanoseconds>(system_clock::now().time_since_epoch()).count();
}

uint64_t monotonicNanos() {
  using namespace std::chrono;
  return duration_cast<nanoseconds>(steady_clock::now().time_since_epoch()).count();
}

std::string nowString() { return stamp("%Y-%m-%d %H:%M:%S", true); }

}  // namespace pccl
