#include "env.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>

extern char** environ;

namespace pccl {

LaunchEnvironments::LaunchEnvironments() {
  for (char** e = environ; e && *e; ++e) {
    const char* eq = std::strchr(*e, '=');
    if (!eq) continue;
    vars_.emplace(std::string(*e, eq - *e), std::string(eq + 1));
  }
}

LaunchEnvironments& LaunchEnvironments::instance() {
  static LaunchEnvironments inst;
  return inst;
}

std::string LaunchEnvironments::getEnv(const std::string& name) {
  auto& s = instance();
  std::lock_guard<std::mutex> g(s.mu_);
  auto it = s.vars_.find(name);
  return it == s.vars_.end() ? std::string() : it->second;
}

bool LaunchEnvironments::has(const std::string& name) {
  auto& s = instance();
  std::lock_guard<std::mutex> g(s.mu_);
  return s.vars_.count(name) != 0;
}

void LaunchEnvironments::registerOpt(const std::string& name, const std::string& help) {
  auto& s = instance();
  std::lock_guard<std::mutex> g(s.mu_);
  auto it = s.opts_.find(name);
  if (it == s.opts_.end()) s.opts_.emplace(name, help);
  else if (!help.empty()) it->second = help;
}

std::vector<std::string> LaunchEnvironments::listOpt() {
  auto& s = instance();
  std::lock_guard<std::mutex> g(s.mu_);
  std::vector<std::string> out;
  for (auto& kv : s.opts_) out.push_back(kv.first);
  return out;
}

std::string LaunchEnvironments::helpOf(const std::string& name) {
  auto& s = instance();
  std::lock_guard<std::mutex> g(s.mu_);
  auto it = s.opts_.find(name);
  return it == s.opts_.end() ? std::string() : it->second;
}

void LaunchEnvironments::setOverride(const std::string& name, const std::string& value) {
  auto& s = instance();
  std::lock_guard<std::mutex> g(s.mu_);
  s.vars_[name] = value;
}

int64_t LaunchEnvironments::getInt(const std::string& name, int64_t dflt) {
  std::string v = getEnv(name);
  if (v.empty()) return dflt;
  char* end = nullptr;
  long long x = std::strtoll(v.c_str(), &end, 0);
  return (end && *end == '\0') ? x : dflt;
}

double LaunchEnvironments::getDouble(const std::string& name, double dflt) {
  std::string v = getEnv(name);
  if (v.empty()) return dflt;
  char* end = nullptr;
  double x = std::strtod(v.c_str(), &end);
  return (end && *end == '\0') ? x : dflt;
}

bool LaunchEnvironments::getBool(const std::string& name, bool dflt) {
  std::string v = getEnv(name);
  if (v.empty()) return dflt;
  std::transform(v.begin(), v.end(), v.begin(), ::tolower);
  if (v == "1" || v == "true" || v == "yes" || v == "on") return true;
  if (v == "0" || v == "false" || v == "no" || v == "off") return false;
  return dflt;
}

std::string LaunchEnvironments::getStr(const std::string& name, const std::string& dflt) {
  std::string v = getEnv(name);
  return v.empty() ? dflt : v;
}

void registerBuiltinOptions() {
  using L = LaunchEnvironments;
  L::registerOpt("PCCL_LOG_LEVEL", "TRACE|DEBUG|INFO|WARN|ERROR|CRITICAL (default WARN)");
  L::registerOpt("PCCL_LOG_TO_TERMINAL", "1/true: also log to stderr");
  L::registerOpt("PCCL_LOG_FILENAME", "log file name under PCCL_LOG_DIR (default <launch time>.log)");
  L::registerOpt("PCCL_LOG_DIR", "directory of the log file (default /tmp/pccl/log)");
  L::registerOpt("PCCL_DISABLE_IB", "set: never try the verbs transport");
  L::registerOpt("PCCL_IB_DEVICE", "verbs device name");
  L::registerOpt("PCCL_IB_GID_INDEX", "verbs GID index (default 0)");
  L::registerOpt("PCCL_IB_PORT_NUM", "verbs port number (default 1)");
  L::registerOpt("PCCL_WORKSPACE_MB", "symmetric workspace per rank in MiB (default 256)");
  L::registerOpt("PCCL_LANES", "workspace lanes: programs on different lanes may run at once on different streams (default 2)");
  L::registerOpt("PCCL_HEAP_ALIGN_MB", "size/alignment unit of the symmetric heap in MiB (default: recommended multicast granularity; 0 = 2 MiB)");
  L::registerOpt("PCCL_NVLS", "0: do not bind the heap to an NVLS multicast object");
  L::registerOpt("PCCL_NO_COOP", "1: launch CTA-pair kernels without the cooperative attribute (profiler replays)");
  L::registerOpt("PCCL_GEMM_PAIR", "0: single-CTA GEMM tiles instead of CTA pairs");
  L::registerOpt("PCCL_CACHE_DIR", "directory of the synthesised-schedule cache (default ~/.cache/pccl_b200)");
  L::registerOpt("PCCL_MAX_SMS", "upper bound on CTAs a collective may use (default 32)");
  L::registerOpt("PCCL_RESIDENT_IDLE_MS", "the resident interpreter kernel leaves after this long without work (default 20)");
  L::registerOpt("PCCL_IBVERBS_LIB", "library to load the verbs API from (default libibverbs.so.1; tests name a stand-in)");
  L::registerOpt("PCCL_LL", "0 keeps all-reduces of up to 64 KiB off the flag-in-data (low-latency) path (default 1)");
  L::registerOpt("PCCL_AG_TAIL", "all-gather GEMM: tiles left to the copy CTAs once their rows are sent (default -1: from a cost model; 0: none)");
  L::registerOpt("PCCL_EXEC_DELAY_US", "testing aid: the CPU executor of rank PCCL_EXEC_DELAY_RANK sleeps this long before every instruction");
  L::registerOpt("PCCL_EXEC_DELAY_RANK", "testing aid: the rank that PCCL_EXEC_DELAY_US slows down (default none)");
  L::registerOpt("PCCL_HANDLE_TYPE", "fabric: also export GPU heap allocations as fabric handles inside the handle document (needs an IMEX channel; falls back to POSIX descriptors)");
  L::registerOpt("PCCL_GEMM_DYNAMIC", "0: the CTA-pair GEMM kernels walk fixed round-robin tile lists instead of drawing tiles at run time");
  L::registerOpt("PCCL_GROUPED_RAGGED", "0: the grouped GEMM keeps rows on the M side of the tile even when the output features are a multiple of 256");
  L::registerOpt("PCCL_CUDA_DRIVER_LIB", "library to load the CUDA driver API from (default libcuda.so.1; tests name a stand-in)");
  L::registerOpt("PCCL_CHANNELS", "default channel count of schedules generated by pccl.lang.build (default 1)");
  L::registerOpt("PCCL_SPIN_LIMIT", "bounded-wait budget of device-side waits, in nanoseconds (default 2e9)");
  L::registerOpt("PCCL_WAIT_TIMEOUT_MS", "bounded-wait budget of host executors in ms (default 30000)");
  L::registerOpt("PCCL_TRANSPORT", "nvls|p2p|shm|tcp: force a transport");
  L::registerOpt("PCCL_TRACE", "1: record per-instruction timestamps");
  L::registerOpt("PCCL_BOUNDS_CHECK", "1: validate every instruction's ranges before running it");
  L::registerOpt("PCCL_HEARTBEAT_MS", "control-plane heartbeat period in ms (default 200)");
  L::registerOpt("PCCL_HEARTBEAT_MISSES", "missed heartbeats before a node is declared gone (default 10)");
  L::registerOpt("PCCL_HOST_ID", "override the host identity used for same-host detection");
}

}  // namespace pccl
