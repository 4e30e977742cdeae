#include "shm_device.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <stdexcept>

#include "../common/clock.h"
#include "../common/json.h"
#include "../common/log.h"

namespace pccl {

static std::atomic<uint64_t> g_seq{0};

CpuDevice::~CpuDevice() {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& kv : segs_) {
    ::munmap(kv.first, kv.second.bytes);
    if (kv.second.owner) ::shm_unlink(kv.second.name.c_str());
  }
  segs_.clear();
}

void* CpuDevice::allocate(size_t bytes) {
  std::string unused;
  return allocateIpcBuffer(bytes, &unused);
}

void* CpuDevice::allocateIpcBuffer(size_t bytes, std::string* handle) {
  if (bytes == 0) throw std::runtime_error("cpu device: zero-size allocation");
  std::string name = "/pccl." + std::to_string(::getpid()) + "." + std::to_string(g_seq.fetch_add(1)) + "." +
                     std::to_string(monotonicNanos() & 0xffffff);
  int fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) throw std::runtime_error("cpu device: shm_open(" + name + ") failed: " + std::strerror(errno));
  if (::ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
    ::close(fd);
    ::shm_unlink(name.c_str());
    throw std::runtime_error("cpu device: ftruncate failed (is /dev/shm large enough?)");
  }
  void* p = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) {
    ::shm_unlink(name.c_str());
    throw std::runtime_error("cpu device: mmap failed");
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    segs_[p] = Seg{bytes, name, true};
  }
  Json h = Json::object();
  h.set("filename", name);
  h.set("size", static_cast<uint64_t>(bytes));
  if (handle) *handle = h.dump();
  return p;
}

void* CpuDevice::mapBuffer(const std::string& handle) {
  Json h = Json::parse(handle);
  std::string name = h["filename"].asString();
  size_t bytes = static_cast<size_t>(h["size"].asInt());
  if (name.empty() || bytes == 0) throw std::runtime_error("cpu device: malformed shm handle");
  int fd = ::shm_open(name.c_str(), O_RDWR, 0600);
  if (fd < 0) throw std::runtime_error("cpu device: cannot open peer segment " + name);
  void* p = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  if (p == MAP_FAILED) throw std::runtime_error("cpu device: mmap of peer segment failed");
  std::lock_guard<std::mutex> g(mu_);
  segs_[p] = Seg{bytes, name, false};
  return p;
}

void CpuDevice::unmapBuffer(void* ptr) { deallocate(ptr); }

void CpuDevice::deallocate(void* ptr) {
  Seg s;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = segs_.find(ptr);
    if (it == segs_.end()) return;
    s = it->second;
    segs_.erase(it);
  }
  ::munmap(ptr, s.bytes);
  if (s.owner) ::shm_unlink(s.name.c_str());
}

void registerCpuDevice() {
  if (!getDev("cpu")) regDev("cpu", std::make_shared<CpuDevice>());
}

}  // namespace pccl
