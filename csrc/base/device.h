// Device plugin interface: allocator + intra-host sharing + remote communication.
//
// Mirrors the three mix-ins of the reference (include/base/device.h:8-40: AllocatorBase,
// RemoteCommunicatorBase, IpcCommunicatorBase, joined in DeviceBase) and its regDev/getDev
// registry (csrc/base/device.cc:65-73, where getDev always throws).  Every method has a
// "not available" default so a plugin implements only what its hardware can do.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace pccl {

class AllocatorBase {
 public:
  virtual ~AllocatorBase() = default;
  virtual bool allocatorAvailable() { return false; }
  virtual void* allocate(size_t bytes);
  virtual void deallocate(void* ptr);
};

// Sharing memory among processes of one host (POSIX shm for CPU, VMM handles for CUDA).
class IpcCommunicatorBase {
 public:
  virtual ~IpcCommunicatorBase() = default;
  virtual bool IPCAvailable() { return false; }
  // Allocates a shareable buffer; *handle receives a JSON document a peer passes to mapBuffer().
  virtual void* allocateIpcBuffer(size_t bytes, std::string* handle);
  virtual void* mapBuffer(const std::string& handle);
  virtual void unmapBuffer(void* ptr);
};

// Moving bytes to a process that cannot map our memory (other host, or forced by PCCL_TRANSPORT).
class RemoteCommunicatorBase {
 public:
  virtual ~RemoteCommunicatorBase() = default;
  virtual bool remoteCommAvailable() { return false; }
  virtual std::string activate();                                   // returns our endpoint handle
  virtual uint32_t regBuffer(void* ptr, size_t bytes);              // returns a local key
  virtual void unregBuffer(uint32_t key);
  virtual void regRemoteHandle(int peer, const std::string& handle);
  virtual void connect(int peer);
  virtual void disconnect(int peer);
  // Data plane.  put: `bytes` from local `src` into the peer's registered buffer `remote_key` at `remote_off`.
  // signal: add `add` to the peer's signal word `slot`; it becomes visible after every put issued before it to the
  // same peer.  Both return false when the peer cannot be reached (the executor reports ST_PEER_GONE).
  virtual bool put(int peer, uint32_t remote_key, uint64_t remote_off, const void* src, uint64_t bytes);
  virtual bool signal(int peer, uint32_t slot, uint64_t add);
  virtual uint64_t bytesSent() const { return 0; }
  virtual uint64_t bytesReceived() const { return 0; }
};

class DeviceBase : public AllocatorBase, public IpcCommunicatorBase, public RemoteCommunicatorBase {
 public:
  virtual std::string name() const = 0;
};

void regDev(const std::string& type, std::shared_ptr<DeviceBase> dev);
std::shared_ptr<DeviceBase> getDev(const std::string& type);   // nullptr if unknown
std::vector<std::string> listDevs();

}  // namespace pccl
