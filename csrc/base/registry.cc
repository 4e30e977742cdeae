#include "registry.h"

#include <stdexcept>

namespace pccl {

TypeRegistry::State& TypeRegistry::state() {
  static State s;
  return s;
}

GeneralType TypeRegistry::registerType(Namespace ns, const std::string& name) {
  State& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  auto it = s.ids[ns].find(name);
  if (it != s.ids[ns].end()) return it->second;
  if (s.by_id[ns].size() >= 256) throw std::runtime_error("TypeRegistry: namespace full");
  GeneralType id = static_cast<GeneralType>(s.by_id[ns].size());
  s.by_id[ns].push_back(name);
  s.ids[ns][name] = id;
  return id;
}

bool TypeRegistry::lookup(Namespace ns, const std::string& name, GeneralType* id) {
  State& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  auto it = s.ids[ns].find(name);
  if (it == s.ids[ns].end()) return false;
  if (id) *id = it->second;
  return true;
}

std::string TypeRegistry::nameOf(Namespace ns, GeneralType id) {
  State& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  return id < s.by_id[ns].size() ? s.by_id[ns][id] : std::string();
}

std::vector<std::string> TypeRegistry::names(Namespace ns) {
  State& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  return s.by_id[ns];
}

void TypeRegistry::setCompatible(const std::string& executor, Namespace ns, const std::string& type) {
  State& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  s.compat[executor].insert({static_cast<int>(ns), type});
  s.reverse[{static_cast<int>(ns), type}].insert(executor);
}

bool TypeRegistry::isCompatible(const std::string& executor, Namespace ns, const std::string& type) {
  State& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  auto it = s.compat.find(executor);
  return it != s.compat.end() && it->second.count({static_cast<int>(ns), type}) != 0;
}

std::vector<std::string> TypeRegistry::executorsFor(Namespace ns, const std::string& type) {
  State& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  auto it = s.reverse.find({static_cast<int>(ns), type});
  if (it == s.reverse.end()) return {};
  return std::vector<std::string>(it->second.begin(), it->second.end());
}

}  // namespace pccl
