// CUDA device plugin: VMM allocations that peers on the same host map over NVLink, plus the NVLS
// multicast object that gives the same memory a second, switch-reduced address.
//
// Counterpart of the reference's CudaDevice (csrc/plugins/cuda_executor/device.cc:53-196:
// cuMemCreate -> cuMemAddressReserve -> cuMemMap -> cuMemSetAccess -> export as a FABRIC handle;
// the importer maps but never calls cuMemSetAccess, and deallocate unmaps with the unaligned size)
// and of its empty symmetric_memory.h.  B200-first choices:
//   * handles are POSIX file descriptors passed over an AF_UNIX socket (SCM_RIGHTS): a fabric
//     handle needs an IMEX domain, which one NVSwitch box does not need and may not have;
//   * the importer sets RW access for its own device; sizes are kept per mapping;
//   * cuMulticastCreate / AddDevice / BindMem map the heap a second time for multimem.* PTX.
// The driver API is resolved at run time from libcuda.so.1, so the library loads (and its host
// paths work) on a machine without a GPU.
#pragma once
#include <atomic>
#include <map>
#include <mutex>
#include <thread>

#include "../base/device.h"

namespace pccl {

class CudaDevice : public DeviceBase {
 public:
  CudaDevice();
  ~CudaDevice() override;
  std::string name() const override { return "cuda"; }
  bool allocatorAvailable() override;
  void* allocate(size_t bytes) override;
  void deallocate(void* ptr) override;
  bool IPCAvailable() override { return allocatorAvailable(); }
  void* allocateIpcBuffer(size_t bytes, std::string* handle) override;
  void* mapBuffer(const std::string& handle) override;
  void unmapBuffer(void* ptr) override;

  // ---- NVLS multicast ------------------------------------------------------------------------
  // The state of one multicast object lives with its owner (an Engine), not with the device: the
  // device object is process-wide, and several engines of one process (the old and the new engine
  // around an elastic recovery, a world-of-one helper engine, a test fixture) each bind their own
  // heap.  Releasing one object must leave every other mapping alone.
  struct McObject {
    unsigned long long handle = 0;
    size_t bytes = 0;
    void* va = nullptr;        // multicast address of the bound heap
    bool bound = false;
    void* local = nullptr;     // the allocation that is bound
    uint64_t export_id = 0;    // creator side: id under which the fd server hands the object out
  };
  bool multicastSupported();
  size_t multicastGranularity(int num_devices, size_t bytes, bool recommended = false);
  // Rank 0: create the object for `num_devices` GPUs; returns a handle document for the others.
  std::string multicastCreate(size_t bytes, int num_devices, McObject* mc);
  // Every rank (rank 0 passes its own document): import and add this process's device.
  void multicastJoin(const std::string& handle, McObject* mc);
  // After every rank has joined: bind the local allocation `local_ptr` (from allocateIpcBuffer)
  // and map the object; returns the multicast address of the heap.
  void* multicastBind(void* local_ptr, McObject* mc);
  // Unmaps, unbinds and releases `mc` only; a second call is a no-op.
  void multicastRelease(McObject* mc);

  // Asks the handle server at `sock` for allocation `id` with `token`; true when a descriptor came back (it is
  // closed again).  For tests of the server's checks.
  static bool probeFdServer(const std::string& sock, uint64_t id, const std::string& token);
  uint64_t refusedRequests() const { return refused_.load(); }

  size_t allocatedSize(void* ptr);
  int deviceOrdinal();
  static std::string lastError();

 private:
  struct Alloc {
    unsigned long long handle = 0;
    size_t bytes = 0;
    uint64_t id = 0;
    int fd = -1;          // exported fd (owner side), kept for the fd server
    bool imported = false;
  };
  void startFdServer();
  void fdServerLoop();
  void* mapHandle(unsigned long long h, size_t bytes);

  std::mutex mu_;
  std::map<void*, Alloc> allocs_;
  std::map<uint64_t, int> exported_fds_;   // alloc id -> fd
  std::atomic<uint64_t> next_id_{1};
  std::string sock_name_;
  int server_fd_ = -1;
  std::thread server_;
  std::atomic<bool> serving_{false};
  std::atomic<uint64_t> refused_{0};
  std::string token_;                      // 128 random bits; a request for an fd must carry them
};

void registerCudaDevice();   // idempotent; registers even without a GPU (allocatorAvailable()==false)

}  // namespace pccl
