// Environment snapshot and option registry.
//
// Capability parity with the reference's LaunchEnvironments (include/common/environ.h:11-37,
// csrc/common/environ.cc:8-29): the process environment is snapshotted once, getEnv() answers
// from the snapshot ("" when unset), and components register the option names they understand so
// that Python can list them.  Additions: typed getters with defaults, a per-option help string,
// and setOverride() so tests and the Python layer can change an option after start-up.
#pragma once
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace pccl {

class LaunchEnvironments {
 public:
  static LaunchEnvironments& instance();
  static std::string getEnv(const std::string& name);
  static void registerOpt(const std::string& name, const std::string& help = "");
  static std::vector<std::string> listOpt();
  static std::string helpOf(const std::string& name);
  static void setOverride(const std::string& name, const std::string& value);

  static bool has(const std::string& name);
  static int64_t getInt(const std::string& name, int64_t dflt);
  static double getDouble(const std::string& name, double dflt);
  static bool getBool(const std::string& name, bool dflt);
  static std::string getStr(const std::string& name, const std::string& dflt);

 private:
  LaunchEnvironments();
  std::mutex mu_;
  std::map<std::string, std::string> vars_;
  std::map<std::string, std::string> opts_;
};

// Registers every option of the library (idempotent).
void registerBuiltinOptions();

}  // namespace pccl
