#include "device.h"

#include <map>
#include <mutex>
#include <stdexcept>

#include "registry.h"

namespace pccl {

static std::runtime_error na(const char* what) {
  return std::runtime_error(std::string("device: ") + what + " is not available on this device");
}

void* AllocatorBase::allocate(size_t) { throw na("allocate"); }
void AllocatorBase::deallocate(void*) { throw na("deallocate"); }
void* IpcCommunicatorBase::allocateIpcBuffer(size_t, std::string*) { throw na("allocateIpcBuffer"); }
void* IpcCommunicatorBase::mapBuffer(const std::string&) { throw na("mapBuffer"); }
void IpcCommunicatorBase::unmapBuffer(void*) { throw na("unmapBuffer"); }
std::string RemoteCommunicatorBase::activate() { throw na("activate"); }
uint32_t RemoteCommunicatorBase::regBuffer(void*, size_t) { throw na("regBuffer"); }
void RemoteCommunicatorBase::unregBuffer(uint32_t) { throw na("unregBuffer"); }
void RemoteCommunicatorBase::regRemoteHandle(int, const std::string&) { throw na("regRemoteHandle"); }
void RemoteCommunicatorBase::connect(int) { throw na("connect"); }
void RemoteCommunicatorBase::disconnect(int) { throw na("disconnect"); }
bool RemoteCommunicatorBase::put(int, uint32_t, uint64_t, const void*, uint64_t) { return false; }
bool RemoteCommunicatorBase::signal(int, uint32_t, uint64_t) { return false; }

namespace {
std::mutex& mu() { static std::mutex m; return m; }
std::map<std::string, std::shared_ptr<DeviceBase>>& table() {
  static std::map<std::string, std::shared_ptr<DeviceBase>> t;
  return t;
}
}  // namespace

void regDev(const std::string& type, std::shared_ptr<DeviceBase> dev) {
  TypeRegistry::registerDeviceType(type);
  std::lock_guard<std::mutex> g(mu());
  table()[type] = std::move(dev);
}

std::shared_ptr<DeviceBase> getDev(const std::string& type) {
  std::lock_guard<std::mutex> g(mu());
  auto it = table().find(type);
  return it == table().end() ? nullptr : it->second;
}

std::vector<std::string> listDevs() {
  std::lock_guard<std::mutex> g(mu());
  std::vector<std::string> out;
  for (auto& kv : table()) out.push_back(kv.first);
  return out;
}

}  // namespace pccl
