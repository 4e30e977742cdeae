#include "cuda_device.h"

#include <cuda.h>
#include <dlfcn.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

#include "../cluster/wire.h"
#include "../common/env.h"
#include "../common/hex.h"
#include "../common/json.h"
#include "../common/log.h"

namespace pccl {

namespace {

// ---- driver API, resolved lazily -------------------------------------------------------------
struct Driver {
  bool ok = false;
  std::string why;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*CtxGetDevice)(CUdevice*) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
};

Driver& drv() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    // PCCL_CUDA_DRIVER_LIB names another library with the same entry points: the CPU tests point it at a
    // stand-in driver that backs "device" allocations with memfd pages, which exercises handle passing,
    // peer mapping and the multicast bookkeeping on a machine without a GPU.
    std::string libname = LaunchEnvironments::getStr("PCCL_CUDA_DRIVER_LIB", "libcuda.so.1");
    void* lib = ::dlopen(libname.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
      d.why = libname + " not found (no NVIDIA driver on this machine)";
      return;
    }
    using GetProc = CUresult (*)(const char*, void**, int, cuuint64_t, CUdriverProcAddressQueryResult*);
    auto getproc = reinterpret_cast<GetProc>(::dlsym(lib, "cuGetProcAddress_v2"));
    auto load = [&](const char* name, void** fn) {
      *fn = nullptr;
      if (getproc) {
        CUdriverProcAddressQueryResult st;
        if (getproc(name, fn, 12040, CU_GET_PROC_ADDRESS_DEFAULT, &st) == CUDA_SUCCESS && *fn) return true;
      }
      *fn = ::dlsym(lib, name);
      return *fn != nullptr;
    };
    bool all = true;
#define PCCL_LOAD(field, sym) all = load(sym, reinterpret_cast<void**>(&d.field)) && all
    PCCL_LOAD(GetErrorString, "cuGetErrorString");
    PCCL_LOAD(CtxGetDevice, "cuCtxGetDevice");
    PCCL_LOAD(DeviceGetAttribute, "cuDeviceGetAttribute");
    PCCL_LOAD(MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    PCCL_LOAD(MemCreate, "cuMemCreate");
    PCCL_LOAD(MemRelease, "cuMemRelease");
    PCCL_LOAD(MemAddressReserve, "cuMemAddressReserve");
    PCCL_LOAD(MemAddressFree, "cuMemAddressFree");
    PCCL_LOAD(MemMap, "cuMemMap");
    PCCL_LOAD(MemUnmap, "cuMemUnmap");
    PCCL_LOAD(MemSetAccess, "cuMemSetAccess");
    PCCL_LOAD(MemExportToShareableHandle, "cuMemExportToShareableHandle");
    PCCL_LOAD(MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    bool mc = true;
#define PCCL_LOAD_MC(field, sym) mc = load(sym, reinterpret_cast<void**>(&d.field)) && mc
    PCCL_LOAD_MC(MulticastCreate, "cuMulticastCreate");
    PCCL_LOAD_MC(MulticastAddDevice, "cuMulticastAddDevice");
    PCCL_LOAD_MC(MulticastBindMem, "cuMulticastBindMem");
    PCCL_LOAD_MC(MulticastUnbind, "cuMulticastUnbind");
    PCCL_LOAD_MC(MulticastGetGranularity, "cuMulticastGetGranularity");
    if (!mc) d.MulticastCreate = nullptr;
    d.ok = all;
    if (!all) d.why = "libcuda.so.1 lacks the virtual memory management API";
  });
  return d;
}

thread_local std::string g_last_error;

void check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return;
  const char* s = nullptr;
  if (drv().GetErrorString) drv().GetErrorString(r, &s);
  g_last_error = std::string(what) + " failed: " + (s ? s : "unknown CUDA error") + " (" + std::to_string(r) + ")";
  throw std::runtime_error("cuda device: " + g_last_error);
}

CUdevice currentDevice() {
  CUdevice dev;
  check(drv().CtxGetDevice(&dev), "cuCtxGetDevice (is a CUDA context current on this thread?)");
  return dev;
}

// PCCL_HANDLE_TYPE=fabric asks for allocations that can ALSO be exported as fabric handles (64 opaque bytes that travel
// in the handle document itself and are valid across the hosts of one NVLink domain, where a file descriptor is not);
// the reference exports them whenever the platform has them (csrc/plugins/cuda_executor/device.cc:105-112, 156-196).
// Where the driver refuses such an allocation (no IMEX channel: any single NVSwitch box) the POSIX descriptor alone is used.
bool wantFabric() {
  const char* v = std::getenv("PCCL_HANDLE_TYPE");
  return v && std::string(v) == "fabric";
}

CUmemAllocationProp allocProp(CUdevice dev, bool fabric = false) {
  CUmemAllocationProp p{};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = static_cast<CUmemAllocationHandleType>(
      CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR | (fabric ? CU_MEM_HANDLE_TYPE_FABRIC : 0));
  return p;
}

size_t alignUp(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

std::string CudaDevice::lastError() { return g_last_error; }

CudaDevice::CudaDevice() {}

CudaDevice::~CudaDevice() {
  serving_.store(false);
  if (server_fd_ >= 0) wire::shutdownFd(server_fd_);
  if (server_.joinable()) server_.join();
  wire::closeFd(server_fd_);
  std::map<void*, Alloc> allocs;
  {
    std::lock_guard<std::mutex> g(mu_);
    allocs.swap(allocs_);
  }
  if (!drv().ok) return;
  for (auto& kv : allocs) {
    CUdeviceptr p = reinterpret_cast<CUdeviceptr>(kv.first);
    drv().MemUnmap(p, kv.second.bytes);
    drv().MemAddressFree(p, kv.second.bytes);
    drv().MemRelease(kv.second.handle);
    if (kv.second.fd >= 0) ::close(kv.second.fd);
  }
}

bool CudaDevice::allocatorAvailable() {
  if (!drv().ok) return false;
  CUdevice dev;
  if (drv().CtxGetDevice(&dev) != CUDA_SUCCESS) return false;
  int vmm = 0;
  drv().DeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev);
  return vmm != 0;
}

int CudaDevice::deviceOrdinal() { return static_cast<int>(currentDevice()); }

void* CudaDevice::mapHandle(unsigned long long h, size_t bytes) {
  CUdevice dev = currentDevice();
  CUdeviceptr va = 0;
  // a mapping whose size allows it is aligned to 512 MiB (or its largest power-of-two divisor), so that the
  // driver is free to back it with its largest pages
  size_t align = 0;
  for (size_t a = 512ull << 20; a >= (2ull << 20); a >>= 1)
    if (bytes % a == 0) { align = a; break; }
  if (drv().MemAddressReserve(&va, bytes, align, 0, 0) != CUDA_SUCCESS)
    check(drv().MemAddressReserve(&va, bytes, 0, 0, 0), "cuMemAddressReserve");
  CUresult r = drv().MemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    drv().MemAddressFree(va, bytes);
    check(r, "cuMemMap");
  }
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = drv().MemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    drv().MemUnmap(va, bytes);
    drv().MemAddressFree(va, bytes);
    check(r, "cuMemSetAccess");
  }
  return reinterpret_cast<void*>(va);
}

void* CudaDevice::allocate(size_t bytes) {
  std::string unused;
  return allocateIpcBuffer(bytes, &unused);
}

void* CudaDevice::allocateIpcBuffer(size_t bytes, std::string* handle) {
  if (!drv().ok) throw std::runtime_error("cuda device: " + drv().why);
  CUdevice dev = currentDevice();
  CUmemAllocationProp prop = allocProp(dev);
  size_t gran = 0;
  check(drv().MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (gran < (2u << 20)) gran = 2u << 20;
  size_t size = alignUp(bytes, gran);
  Alloc a;
  bool fabric = wantFabric();
  if (fabric) {
    CUmemAllocationProp fprop = allocProp(dev, true);
    if (drv().MemCreate(&a.handle, size, &fprop, 0) != CUDA_SUCCESS) {
      PCCL_LOG_WARN("cuda device: the driver refused an allocation with fabric handles; using POSIX descriptors only");
      fabric = false;
    }
  }
  if (!fabric) check(drv().MemCreate(&a.handle, size, &prop, 0), "cuMemCreate");
  a.bytes = size;
  a.id = next_id_.fetch_add(1);
  void* ptr = nullptr;
  std::string fabric_hex;
  try {
    ptr = mapHandle(a.handle, size);
    int fd = -1;
    check(drv().MemExportToShareableHandle(&fd, a.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
          "cuMemExportToShareableHandle");
    a.fd = fd;
    if (fabric) {
      CUmemFabricHandle fh{};
      if (drv().MemExportToShareableHandle(&fh, a.handle, CU_MEM_HANDLE_TYPE_FABRIC, 0) == CUDA_SUCCESS)
        fabric_hex = encodeHex(fh.data, sizeof(fh.data));
      else
        PCCL_LOG_WARN("cuda device: exporting the fabric handle failed; peers will use the POSIX descriptor");
    }
  } catch (...) {
    if (ptr) {
      drv().MemUnmap(reinterpret_cast<CUdeviceptr>(ptr), size);
      drv().MemAddressFree(reinterpret_cast<CUdeviceptr>(ptr), size);
    }
    drv().MemRelease(a.handle);
    throw;
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    allocs_[ptr] = a;
    exported_fds_[a.id] = a.fd;
  }
  startFdServer();
  Json h = Json::object();
  h.set("size", static_cast<uint64_t>(size));
  h.set("id", a.id);
  h.set("pid", static_cast<int64_t>(::getpid()));
  h.set("sock", sock_name_);
  h.set("token", token_);
  h.set("device", static_cast<int>(dev));
  if (!fabric_hex.empty()) h.set("fabric", fabric_hex);
  if (handle) *handle = h.dump();
  return ptr;
}

// The handle-passing socket lives in the abstract AF_UNIX namespace, which every process of the network
// namespace can reach, and allocation ids are small integers.  So a request is served only when (a) the
// kernel says the peer runs under our own user id (SO_PEERCRED) and (b) it carries the 128-bit random token
// that travels in the handle document (which peers receive over the job's own rendezvous).  Anything else
// gets an answer without a descriptor.
void CudaDevice::startFdServer() {
  std::lock_guard<std::mutex> g(mu_);
  if (serving_.load()) return;
  unsigned char rnd[16];
  bool have = false;
  if (FILE* f = std::fopen("/dev/urandom", "rb")) {
    have = std::fread(rnd, 1, sizeof(rnd), f) == sizeof(rnd);
    std::fclose(f);
  }
  if (!have) throw std::runtime_error("cuda device: no random source for the handle token");
  token_ = encodeHex(rnd, sizeof(rnd));
  sock_name_ = "pccl-vmm-" + std::to_string(::getpid()) + "-" + token_.substr(0, 8);
  server_fd_ = wire::unixListen(sock_name_);
  if (server_fd_ < 0) throw std::runtime_error("cuda device: cannot create the handle-passing socket");
  serving_.store(true);
  server_ = std::thread([this] { fdServerLoop(); });
}

namespace {
struct FdRequest {
  uint64_t id;
  char token[32];     // hex digits of the 128-bit token
};
bool sameToken(const char* a, const std::string& b) {
  if (b.size() != 32) return false;
  unsigned char diff = 0;
  for (int i = 0; i < 32; ++i) diff |= static_cast<unsigned char>(a[i] ^ b[i]);   // no early exit
  return diff == 0;
}
}  // namespace

void CudaDevice::fdServerLoop() {
  while (serving_.load()) {
    int c = wire::acceptOne(server_fd_, 100);
    if (c < 0) continue;
    FdRequest rq{};
    if (wire::recvAll(c, &rq, sizeof(rq))) {
      int fd = -1;
      long uid = wire::peerUid(c);
      bool trusted = uid >= 0 && static_cast<uid_t>(uid) == ::geteuid() && sameToken(rq.token, token_);
      if (trusted) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = exported_fds_.find(rq.id);
        if (it != exported_fds_.end()) fd = it->second;
      } else {
        refused_.fetch_add(1);
        PCCL_LOG_WARN("cuda device: refused a memory-handle request (peer uid %ld, token %s)", uid,
                      sameToken(rq.token, token_) ? "ok" : "wrong");
      }
      wire::sendFd(c, fd, rq.id);
    }
    wire::closeFd(c);
  }
}

static int fetchFd(const std::string& sock, uint64_t id, const std::string& token) {
  int c = wire::unixConnect(sock, 10000);
  if (c < 0) throw std::runtime_error("cuda device: cannot reach peer handle socket " + sock);
  FdRequest rq{};
  rq.id = id;
  std::memcpy(rq.token, token.data(), std::min<size_t>(token.size(), sizeof(rq.token)));
  int fd = -1;
  uint64_t tag = 0;
  bool ok = wire::sendAll(c, &rq, sizeof(rq)) && wire::recvFd(c, &fd, &tag);
  wire::closeFd(c);
  if (!ok || fd < 0 || tag != id) throw std::runtime_error("cuda device: peer did not hand over the memory handle");
  return fd;
}

bool CudaDevice::probeFdServer(const std::string& sock, uint64_t id, const std::string& token) {
  try {
    int fd = fetchFd(sock, id, token);
    ::close(fd);
    return true;
  } catch (const std::exception&) {
    return false;
  }
}

void* CudaDevice::mapBuffer(const std::string& handle) {
  if (!drv().ok) throw std::runtime_error("cuda device: " + drv().why);
  Json h = Json::parse(handle);
  size_t size = static_cast<size_t>(h["size"].asInt());
  uint64_t id = static_cast<uint64_t>(h["id"].asInt());
  Alloc a;
  bool imported = false;
  if (wantFabric() && h.contains("fabric")) {
    // the 64 bytes came with the document: no descriptor to fetch, and the owner may be on another host of the domain
    CUmemFabricHandle fh{};
    if (decodeHex(fh.data, sizeof(fh.data), h["fabric"].asString()) &&
        drv().MemImportFromShareableHandle(&a.handle, &fh, CU_MEM_HANDLE_TYPE_FABRIC) == CUDA_SUCCESS)
      imported = true;
    else
      PCCL_LOG_WARN("cuda device: importing the fabric handle failed; asking the owner for a POSIX descriptor");
  }
  if (!imported) {
    int fd = fetchFd(h["sock"].asString(), id, h["token"].asString());
    CUresult r = drv().MemImportFromShareableHandle(&a.handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    check(r, "cuMemImportFromShareableHandle");
  }
  a.bytes = size;
  a.imported = true;
  void* ptr = nullptr;
  try {
    ptr = mapHandle(a.handle, size);
  } catch (...) {
    drv().MemRelease(a.handle);
    throw;
  }
  std::lock_guard<std::mutex> g(mu_);
  allocs_[ptr] = a;
  return ptr;
}

void CudaDevice::unmapBuffer(void* ptr) { deallocate(ptr); }

void CudaDevice::deallocate(void* ptr) {
  Alloc a;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = allocs_.find(ptr);
    if (it == allocs_.end()) return;
    a = it->second;
    allocs_.erase(it);
    exported_fds_.erase(a.id);
  }
  CUdeviceptr p = reinterpret_cast<CUdeviceptr>(ptr);
  drv().MemUnmap(p, a.bytes);
  drv().MemAddressFree(p, a.bytes);
  drv().MemRelease(a.handle);
  if (a.fd >= 0) ::close(a.fd);
}

size_t CudaDevice::allocatedSize(void* ptr) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = allocs_.find(ptr);
  return it == allocs_.end() ? 0 : it->second.bytes;
}

// ---- multicast ---------------------------------------------------------------------------------
bool CudaDevice::multicastSupported() {
  if (!drv().ok || !drv().MulticastCreate) return false;
  CUdevice dev;
  if (drv().CtxGetDevice(&dev) != CUDA_SUCCESS) return false;
  int mc = 0;
  drv().DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev);
  return mc != 0;
}

size_t CudaDevice::multicastGranularity(int num_devices, size_t bytes, bool recommended) {
  CUmulticastObjectProp p{};
  p.numDevices = static_cast<unsigned>(num_devices);
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g = 0;
  check(drv().MulticastGetGranularity(&g, &p, recommended ? CU_MULTICAST_GRANULARITY_RECOMMENDED : CU_MULTICAST_GRANULARITY_MINIMUM),
        "cuMulticastGetGranularity");
  return g;
}

std::string CudaDevice::multicastCreate(size_t bytes, int num_devices, McObject* mc) {
  if (!multicastSupported()) throw std::runtime_error("cuda device: multicast is not supported here");
  if (mc->handle) throw std::runtime_error("cuda device: this owner already holds a multicast object");
  CUmulticastObjectProp p{};
  p.numDevices = static_cast<unsigned>(num_devices);
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  check(drv().MulticastCreate(&h, &p), "cuMulticastCreate");
  int fd = -1;
  CUresult r = drv().MemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    drv().MemRelease(h);
    check(r, "cuMemExportToShareableHandle(multicast)");
  }
  uint64_t id = next_id_.fetch_add(1);
  {
    std::lock_guard<std::mutex> g(mu_);
    exported_fds_[id] = fd;
  }
  mc->handle = h;
  mc->bytes = bytes;
  mc->export_id = id;
  startFdServer();
  Json j = Json::object();
  j.set("size", static_cast<uint64_t>(bytes));
  j.set("id", id);
  j.set("pid", static_cast<int64_t>(::getpid()));
  j.set("sock", sock_name_);
  j.set("token", token_);
  j.set("num_devices", num_devices);
  return j.dump();
}

void CudaDevice::multicastJoin(const std::string& handle, McObject* mc) {
  Json j = Json::parse(handle);
  size_t bytes = static_cast<size_t>(j["size"].asInt());
  const bool mine = j["pid"].asInt() == static_cast<int64_t>(::getpid()) && mc->handle != 0 &&
                    mc->export_id == static_cast<uint64_t>(j["id"].asInt());
  if (!mine) {
    if (mc->handle) throw std::runtime_error("cuda device: this owner already holds a multicast object");
    int fd = fetchFd(j["sock"].asString(), static_cast<uint64_t>(j["id"].asInt()), j["token"].asString());
    CUmemGenericAllocationHandle h;
    CUresult r = drv().MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    check(r, "cuMemImportFromShareableHandle(multicast)");
    mc->handle = h;
    mc->bytes = bytes;
  }
  check(drv().MulticastAddDevice(mc->handle, currentDevice()), "cuMulticastAddDevice");
}

void* CudaDevice::multicastBind(void* local_ptr, McObject* mc) {
  Alloc a;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = allocs_.find(local_ptr);
    if (it == allocs_.end()) throw std::runtime_error("cuda device: multicastBind of an unknown allocation");
    a = it->second;
  }
  if (!mc->handle) throw std::runtime_error("cuda device: multicastBind before multicastJoin");
  if (a.bytes < mc->bytes) throw std::runtime_error("cuda device: allocation smaller than the multicast object");
  check(drv().MulticastBindMem(mc->handle, 0, a.handle, 0, mc->bytes, 0), "cuMulticastBindMem");
  mc->bound = true;
  mc->local = local_ptr;
  mc->va = mapHandle(mc->handle, mc->bytes);
  return mc->va;
}

void CudaDevice::multicastRelease(McObject* mc) {
  if (!drv().ok || !mc || mc->handle == 0) return;
  if (mc->va) {
    CUdeviceptr p = reinterpret_cast<CUdeviceptr>(mc->va);
    drv().MemUnmap(p, mc->bytes);
    drv().MemAddressFree(p, mc->bytes);
  }
  if (mc->bound) {
    CUdevice dev;
    if (drv().CtxGetDevice(&dev) == CUDA_SUCCESS) drv().MulticastUnbind(mc->handle, dev, 0, mc->bytes);
  }
  drv().MemRelease(mc->handle);
  if (mc->export_id) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = exported_fds_.find(mc->export_id);
    if (it != exported_fds_.end()) {
      if (it->second >= 0) ::close(it->second);
      exported_fds_.erase(it);
    }
  }
  *mc = McObject{};
}

void registerCudaDevice() {
  if (!getDev("cuda")) regDev("cuda", std::make_shared<CudaDevice>());
}

}  // namespace pccl
