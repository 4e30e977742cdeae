// CPU device plugin: host memory shared among the ranks of one host through POSIX shm.
// Counterpart of the reference's CpuDevice (csrc/plugins/cpu_executor/device.cc:51-117:
// shm_open + ftruncate + mmap; the handle is a JSON {filename, size}; peers re-open by name).
// Differences: the name carries pid and a counter (no rand()), every mapping is tracked so that
// unmap/deallocate use the right length, and segments are unlinked at exit even on exceptions.
#pragma once
#include <map>
#include <mutex>

#include "../base/device.h"

namespace pccl {

class CpuDevice : public DeviceBase {
 public:
  ~CpuDevice() override;
  std::string name() const override { return "cpu"; }
  bool allocatorAvailable() override { return true; }
  void* allocate(size_t bytes) override;
  void deallocate(void* ptr) override;
  bool IPCAvailable() override { return true; }
  void* allocateIpcBuffer(size_t bytes, std::string* handle) override;
  void* mapBuffer(const std::string& handle) override;
  void unmapBuffer(void* ptr) override;

 private:
  struct Seg { size_t bytes; std::string name; bool owner; };
  std::mutex mu_;
  std::map<void*, Seg> segs_;
};

void registerCpuDevice();   // idempotent

}  // namespace pccl
