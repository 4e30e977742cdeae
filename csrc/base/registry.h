// Runtime registry of type ids.
//
// The reference declares a TypeRegistry that hands out one-byte ids in five namespaces
// (primitive, data, compute, device, executor) and records which executor kinds can run which
// type (include/base/registry.h:12-80); its source file is an empty namespace
// (csrc/base/registry.cc:1-5).  Here dtypes, opcodes and reduce ops are compile-time enums
// (instr.h) because device code needs them as constants; the registry keeps the runtime-extensible
// part: device kinds and executor kinds that plugins add at load time, and their compatibility.
#pragma once
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <vector>

namespace pccl {

using GeneralType = unsigned char;

class TypeRegistry {
 public:
  enum Namespace { Primitive = 0, Data, Compute, Device, Executor, kNumNamespaces };

  static GeneralType registerType(Namespace ns, const std::string& name);  // idempotent
  static bool lookup(Namespace ns, const std::string& name, GeneralType* id);
  static std::string nameOf(Namespace ns, GeneralType id);
  static std::vector<std::string> names(Namespace ns);

  static GeneralType registerDeviceType(const std::string& n) { return registerType(Device, n); }
  static GeneralType registerExecutorType(const std::string& n) { return registerType(Executor, n); }
  static std::vector<std::string> getDeviceTypes() { return names(Device); }

  // executor <-> (namespace, type) compatibility, with reverse lookup
  static void setCompatible(const std::string& executor, Namespace ns, const std::string& type);
  static bool isCompatible(const std::string& executor, Namespace ns, const std::string& type);
  static std::vector<std::string> executorsFor(Namespace ns, const std::string& type);

 private:
  struct State {
    std::mutex mu;
    std::map<std::string, GeneralType> ids[kNumNamespaces];
    std::vector<std::string> by_id[kNumNamespaces];
    std::map<std::string, std::set<std::pair<int, std::string>>> compat;
    std::map<std::pair<int, std::string>, std::set<std::string>> reverse;
  };
  static State& state();
};

}  // namespace pccl
