#include "engine.h"

#include <cuda_runtime.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <thread>
#include <fstream>
#include <stdexcept>

#include "common/clock.h"
#include "common/env.h"
#include "common/hash.h"
#include "common/json.h"
#include "common/log.h"
#include "mem/shm_device.h"

namespace pccl {

namespace {
constexpr uint64_t kMiB = 1ull << 20;
uint64_t alignUp(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

std::string readHostId() {
  std::string v = LaunchEnvironments::getEnv("PCCL_HOST_ID");
  if (!v.empty()) return v;
  std::ifstream f("/proc/sys/kernel/random/boot_id");
  std::string id;
  if (f && std::getline(f, id) && !id.empty()) return id;
  char name[256] = {0};
  ::gethostname(name, sizeof(name) - 1);
  return name;
}

void cudaCheck(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("engine: ") + what + ": " + cudaGetErrorString(e));
}

// Device-memory copies and reductions for the host-driven executor.  Worker threads are short-lived, so streams come
// from a small pool; every call makes the engine's device current in the calling thread first.
class CudaMemOps : public MemOps {
 public:
  explicit CudaMemOps(int device) : device_(device) {}
  ~CudaMemOps() override {
    for (cudaStream_t s : pool_) cudaStreamDestroy(s);
  }
  bool copy(void* dst, const void* src, uint64_t bytes) override {
    Lease l(this);
    return l.s && cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, l.s) == cudaSuccess && cudaStreamSynchronize(l.s) == cudaSuccess;
  }
  bool reduce(void* dst, const void* src, uint64_t bytes, uint32_t dtype, uint32_t redop) override {
    Lease l(this);
    return l.s && launchDeviceReduce(dst, src, bytes, dtype, redop, l.s) == 0 && cudaStreamSynchronize(l.s) == cudaSuccess;
  }
  const void* toHost(const void* src, uint64_t bytes) override {
    thread_local std::vector<char> buf;
    if (buf.size() < bytes) buf.resize(bytes);
    Lease l(this);
    if (!l.s || cudaMemcpyAsync(buf.data(), src, bytes, cudaMemcpyDeviceToHost, l.s) != cudaSuccess || cudaStreamSynchronize(l.s) != cudaSuccess)
      return nullptr;
    return buf.data();
  }

 private:
  struct Lease {
    CudaMemOps* o;
    cudaStream_t s = nullptr;
    explicit Lease(CudaMemOps* ops) : o(ops) {
      if (cudaSetDevice(o->device_) != cudaSuccess) return;
      std::lock_guard<std::mutex> g(o->mu_);
      if (!o->pool_.empty()) {
        s = o->pool_.back();
        o->pool_.pop_back();
      } else if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
        s = nullptr;
      }
    }
    ~Lease() {
      if (!s) return;
      std::lock_guard<std::mutex> g(o->mu_);
      o->pool_.push_back(s);
    }
  };
  int device_;
  std::mutex mu_;
  std::vector<cudaStream_t> pool_;
};
}  // namespace

Engine::Engine(int rank, int world) : rank_(rank), world_(world) {
  if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("Engine: need 0 <= rank < world");
  if (world > kMaxRanks) throw std::runtime_error("Engine: world size above the compiled maximum");
  registerBuiltinOptions();
}

Engine::~Engine() {
  try {
    stopResident();
  } catch (...) {
  }
  try {
    exitCluster();
  } catch (...) {
  }
  for (auto& kv : ops_)
    for (auto& dc : kv.second.device_cache) {
      if (dc.second.instrs) cudaFree(dc.second.instrs);
      if (dc.second.starts) cudaFree(dc.second.starts);
    }
  for (auto& t : dtrace_)
    if (t.words) cudaFree(t.words);
  dropPeers();
  if (tcp_) tcp_->shutdown();
  if (verbs_) verbs_->shutdown();
  device_mem_ops_.reset();
  if (shadow_stream_) cudaStreamDestroy(static_cast<cudaStream_t>(shadow_stream_));
  if (shadow_) cudaFreeHost(shadow_);
  delete[] host_signals_;
  if (heap_) {
    auto dev = getDev(device_);
    if (dev) {
      try {
        // only the multicast object that THIS engine created or joined: other engines of the process keep theirs
        if (device_ == "cuda") static_cast<CudaDevice*>(dev.get())->multicastRelease(&mc_);
        dev->deallocate(heap_);
      } catch (...) {
      }
    }
    heap_ = nullptr;
  }
}

void Engine::buildLayout(uint64_t heap_bytes) {
  HeapLayout& L = layout_;
  L.workspace_bytes = static_cast<uint64_t>(LaunchEnvironments::getInt("PCCL_WORKSPACE_MB", 256)) * kMiB;
  L.lanes = static_cast<int>(LaunchEnvironments::getInt("PCCL_LANES", 2));
  if (L.lanes < 1) L.lanes = 1;
  L.signal_off = L.workspace_bytes;
  L.num_signals = 65536;
  L.finish_base = static_cast<uint32_t>(L.num_signals) - kMaxLanes;
  L.turn_base = L.finish_base - kMaxLanes * kMaxRanks;
  if (L.lanes > kMaxLanes) L.lanes = kMaxLanes;
  L.flag_off = L.signal_off + L.num_signals * 8;
  L.flag_bytes = alignUp(8ull * kMaxBlocksPerColl * kMaxRanks * 8, 256 * 1024);
  L.status_off = L.flag_off + L.flag_bytes;
  L.status_bytes = 4096;
  L.ll_off = alignUp(L.status_off + L.status_bytes, 4096);
  L.user_off = alignUp(L.ll_off + kLlLanes * kLlLaneBytes, 2 * kMiB);
  L.total = alignUp(std::max(heap_bytes, L.user_off), 2 * kMiB);
  user_top_ = L.user_off;
}

void Engine::initEngine(const std::string& device, uint64_t heap_bytes) {
  if (initialized_) return;
  registerCpuDevice();
  registerCudaDevice();
  device_ = device;
  if (device_ == "auto") device_ = getDev("cuda")->allocatorAvailable() ? "cuda" : "cpu";
  auto dev = getDev(device_);
  if (!dev) throw std::runtime_error("initEngine: unknown device kind '" + device_ + "'");
  if (!dev->allocatorAvailable()) throw std::runtime_error("initEngine: device '" + device_ + "' is not usable here");
  timeout_ms_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_WAIT_TIMEOUT_MS", 30000));
  spin_limit_ = static_cast<uint64_t>(LaunchEnvironments::getInt("PCCL_SPIN_LIMIT", static_cast<int64_t>(kDefaultSpinLimit)));
  bounds_check_ = LaunchEnvironments::getBool("PCCL_BOUNDS_CHECK", true);
  trace_ = LaunchEnvironments::getBool("PCCL_TRACE", false);
  max_width_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_MAX_SMS", 32));
  exec_delay_us_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_EXEC_DELAY_US", 0));
  exec_delay_rank_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_EXEC_DELAY_RANK", -1));
  host_id_ = readHostId();
  buildLayout(heap_bytes);
  if (device_ == "cuda" && world_ > 1) {
    // Size the heap in units of the RECOMMENDED multicast granularity (the minimum one still binds, but
    // leaves the multicast mapping on small pages); PCCL_HEAP_ALIGN_MB overrides, 0 keeps 2 MiB.
    auto* cdev = static_cast<CudaDevice*>(dev.get());
    size_t g = 0;
    const int64_t forced = LaunchEnvironments::getInt("PCCL_HEAP_ALIGN_MB", -1);
    if (forced > 0) g = static_cast<size_t>(forced) * kMiB;
    else if (forced < 0 && cdev->multicastSupported()) {
      try {
        g = cdev->multicastGranularity(world_, layout_.total, true);
        PCCL_LOG_INFO("multicast granularity: minimum %zu, recommended %zu bytes", cdev->multicastGranularity(world_, layout_.total, false), g);
      } catch (const std::exception&) { g = 0; }
    }
    if (g >= 2 * kMiB && g <= 1024 * kMiB) layout_.total = alignUp(layout_.total, g);
  }
  heap_ = static_cast<char*>(dev->allocateIpcBuffer(layout_.total, &heap_handle_));
  uint64_t ctl = layout_.user_off - layout_.signal_off;
  if (device_ == "cuda") {
    cudaCheck(cudaMemset(heap_ + layout_.signal_off, 0, ctl), "clearing the signal area");
    cudaCheck(cudaDeviceSynchronize(), "synchronize after heap set-up");
  } else {
    std::memset(heap_ + layout_.signal_off, 0, ctl);
  }
  peer_heaps_.assign(world_, nullptr);
  peer_heaps_[rank_] = heap_;
  lane_epochs_.assign(8, 0);
  lane_launches_.assign(64, 0);

  configs_["host_id"] = host_id_;
  configs_["device"] = device_;
  configs_["pid"] = std::to_string(::getpid());
  configs_["heap.bytes"] = std::to_string(layout_.total);
  configs_["ipc." + device_ + ".handle"] = heap_handle_;
  if (device_ == "cpu") {
    tcp_ = std::make_unique<TcpTransport>();
    std::string host = LaunchEnvironments::getStr("PCCL_TCP_HOST", "127.0.0.1");
    tcp_->setAdvertisedHost(host);
    configs_["remote.tcp.endpoint"] = tcp_->activate();
    tcp_key_ = tcp_->regBuffer(heap_, layout_.total);
    tcp_->setSignals(reinterpret_cast<std::atomic<uint64_t>*>(heap_ + layout_.signal_off),
                     static_cast<uint32_t>(layout_.num_signals));
    configs_["remote.tcp.buffer.cpu.key"] = std::to_string(tcp_key_);
    remote_ = tcp_.get();
    remote_key_ = tcp_key_;
  }
  if (device_ == "cuda" && world_ > 1) {
    // a listening socket only; the shadow of the workspace and the host signal words are made when a peer turns out
    // to live on another host (ensureMixedHostResources)
    cudaCheck(cudaGetDevice(&cuda_ordinal_), "cudaGetDevice");
    tcp_ = std::make_unique<TcpTransport>();
    tcp_->setAdvertisedHost(LaunchEnvironments::getStr("PCCL_TCP_HOST", "127.0.0.1"));
    configs_["remote.tcp.endpoint"] = tcp_->activate();
    configs_["remote.tcp.buffer.cuda.key"] = "0";
  }
  std::string why;
  const bool have_verbs = VerbsTransport::probe(&why);
  configs_["remote.verbs.available"] = have_verbs ? "1" : "0";
  configs_["remote.verbs.note"] = why;
  if (device_ == "cpu" && LaunchEnvironments::getEnv("PCCL_TRANSPORT") == "verbs") {
    // asked for by name: without a usable device this is an error, not a silent fall-back
    if (!have_verbs) throw std::runtime_error("initEngine: PCCL_TRANSPORT=verbs, but " + why);
    verbs_ = std::make_unique<VerbsTransport>(rank_, world_);
    verbs_->activate();
    verbs_key_ = verbs_->regBuffer(heap_, layout_.total);
    verbs_->setSignalRegion(verbs_key_, layout_.signal_off, static_cast<uint32_t>(layout_.num_signals));
    configs_["remote.verbs.endpoint"] = verbs_->endpoint();
    configs_["remote.verbs.buffer.cpu.key"] = std::to_string(verbs_key_);
    remote_ = verbs_.get();
    remote_key_ = verbs_key_;
  }
  initialized_ = true;
  PCCL_LOG_INFO("engine: rank %d/%d on %s, heap %llu MiB", rank_, world_, device_.c_str(),
                static_cast<unsigned long long>(layout_.total / kMiB));
}

std::string Engine::exportEndpoint() {
  if (!initialized_) throw std::runtime_error("exportEndpoint: call initEngine first");
  NodeMeta m;
  m.rank_ = rank_;
  m.endpoint_configs_ = configs_;
  return m.serialize();
}

void Engine::dropPeers() {
  auto dev = getDev(device_);
  for (int r = 0; r < static_cast<int>(peer_heaps_.size()); ++r) {
    if (r == rank_ || !peer_heaps_[r]) continue;
    try {
      if (dev) dev->unmapBuffer(peer_heaps_[r]);
    } catch (...) {
    }
    peer_heaps_[r] = nullptr;
  }
  if (tcp_)
    for (int r = 0; r < world_; ++r) tcp_->disconnect(r);
  if (verbs_)
    for (int r = 0; r < world_; ++r)
      if (r != rank_) verbs_->disconnect(r);
}

void Engine::setupPeers(const std::map<int, NodeMeta>& nodes) {
  auto dev = getDev(device_);
  std::string forced = LaunchEnvironments::getEnv("PCCL_TRANSPORT");
  for (auto& kv : nodes) {
    int r = kv.first;
    if (r == rank_ || r < 0 || r >= world_) continue;
    const auto& cfg = kv.second.endpoint_configs_;
    auto get = [&](const std::string& k) {
      auto it = cfg.find(k);
      return it == cfg.end() ? std::string() : it->second;
    };
    if (get("device") != device_) throw std::runtime_error("setupPeers: rank " + std::to_string(r) + " runs on a different device kind");
    bool same_host = get("host_id") == host_id_;
    bool use_tcp = device_ == "cpu" && (forced == "tcp" || forced == "verbs" || !same_host);
    if (!use_tcp) {
      if (!same_host) {
        if (!tcp_) throw std::runtime_error("setupPeers: rank " + std::to_string(r) + " is on another host and this engine has no network transport");
        mixed_hosts_ = true;               // reached through the host shadow of the workspace over TCP
      } else if (!peer_heaps_[r]) {
        peer_heaps_[r] = static_cast<char*>(dev->mapBuffer(get("ipc." + device_ + ".handle")));
      }
    } else {
      if (verbs_) {
        std::string ep = get("remote.verbs.endpoint");
        if (ep.empty()) throw std::runtime_error("setupPeers: rank " + std::to_string(r) + " published no verbs endpoint");
        verbs_->regRemoteHandle(r, ep);
        verbs_->connect(r);
      } else {
        tcp_->regRemoteHandle(r, get("remote.tcp.endpoint"));
        tcp_->connect(r);
      }
    }
  }
  if (device_ == "cuda" && mixed_hosts_) {
    // every signal of the host-driven executor travels over TCP, so every peer needs a connection, also those whose
    // heap is mapped over NVLink
    ensureMixedHostResources();
    for (auto& kv : nodes) {
      int r = kv.first;
      if (r == rank_ || r < 0 || r >= world_) continue;
      auto it = kv.second.endpoint_configs_.find("remote.tcp.endpoint");
      if (it == kv.second.endpoint_configs_.end()) throw std::runtime_error("setupPeers: rank " + std::to_string(r) + " published no TCP endpoint");
      tcp_->regRemoteHandle(r, it->second);
      tcp_->connect(r);
    }
  }
}

void Engine::ensureMixedHostResources() {
  if (shadow_) return;
  cudaCheck(cudaHostAlloc(reinterpret_cast<void**>(&shadow_), layout_.workspace_bytes, cudaHostAllocDefault), "pinned shadow of the workspace");
  host_signals_ = new std::atomic<uint64_t>[layout_.num_signals]();
  cudaStream_t s = nullptr;
  cudaCheck(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "shadow stream");
  shadow_stream_ = s;
  tcp_key_ = tcp_->regBuffer(shadow_, layout_.workspace_bytes);          // the first registration: key 0, as published
  tcp_->setSignals(host_signals_, static_cast<uint32_t>(layout_.num_signals));
  // receiver thread: bytes that arrived in the shadow go on to the same offset of the device heap before the next frame
  // (so before the SIGNAL that follows them) is read
  tcp_->setPutHook([this](uint32_t key, uint64_t off, uint64_t bytes) {
    if (key != tcp_key_ || off + bytes > layout_.workspace_bytes) return;
    cudaStream_t st = static_cast<cudaStream_t>(shadow_stream_);
    if (cudaSetDevice(cuda_ordinal_) != cudaSuccess || cudaMemcpyAsync(heap_ + off, shadow_ + off, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
      PCCL_LOG_ERROR("engine: copying %llu received bytes to the device failed", static_cast<unsigned long long>(bytes));
  });
  device_mem_ops_ = std::make_unique<CudaMemOps>(cuda_ordinal_);
  remote_ = tcp_.get();
  remote_key_ = tcp_key_;
}

void Engine::importEndpoints(const std::vector<std::string>& docs) {
  if (!initialized_) throw std::runtime_error("importEndpoints: call initEngine first");
  std::map<int, NodeMeta> nodes;
  for (auto& d : docs) {
    NodeMeta m;
    if (!NodeMeta::deserialize(d, &m)) throw std::runtime_error("importEndpoints: unreadable endpoint document");
    nodes[m.rank_] = m;
  }
  setupPeers(nodes);
}

void Engine::joinCluster(const std::string& master_endpoint, int timeout_ms) {
  if (!initialized_) throw std::runtime_error("joinCluster: call initEngine first");
  cluster_ = std::make_unique<ClusterManager>(rank_, world_, configs_);
  if (!cluster_->initializeDaemonServer(master_endpoint)) throw std::runtime_error("joinCluster: control plane did not start");
  if (!cluster_->waitForWorld(world_, timeout_ms)) {
    size_t have = cluster_->nodes().size();
    throw std::runtime_error("joinCluster: only " + std::to_string(have) + " of " + std::to_string(world_) + " ranks joined in time");
  }
  setupPeers(cluster_->nodes());
}

void Engine::exitCluster() {
  if (cluster_) {
    cluster_->killDaemonServer();
    cluster_.reset();
  }
}

std::vector<int> Engine::aliveRanks() {
  if (!cluster_) {
    std::vector<int> all;
    for (int r = 0; r < world_; ++r) all.push_back(r);
    return all;
  }
  return cluster_->aliveRanks();
}

std::map<int, int> Engine::resizeWorld() {
  if (!cluster_) throw std::runtime_error("resizeWorld: not in a cluster");
  return cluster_->resizeWorld();
}

std::map<int, int> Engine::lastResize() { return cluster_ ? cluster_->lastResize() : std::map<int, int>(); }

bool Engine::waitForDeparture(int rank, int timeout_ms) { return cluster_ && cluster_->waitForDeparture(rank, timeout_ms); }

void Engine::rebind(int new_rank, int new_world) {
  // Peers are re-mapped by the next importEndpoints/joinCluster; registered programs of the old
  // world size stay registered but cannot run (their world differs).  Everything that counts launches
  // starts again from zero: signal words, barrier flags, status, lane and program epochs -- on a CUDA
  // engine after the device has drained, and with the old world's multicast object released (connect()
  // builds a new one for the new world).
  if (new_world < 1 || new_rank < 0 || new_rank >= new_world || new_world > kMaxRanks)
    throw std::runtime_error("rebind: need 0 <= rank < world <= the compiled maximum");
  std::lock_guard<std::mutex> g(mu_);
  dropPeers();
  char* mine = heap_;
  rank_ = new_rank;
  world_ = new_world;
  peer_heaps_.assign(world_, nullptr);
  peer_heaps_[rank_] = mine;
  const uint64_t ctl = layout_.user_off - layout_.signal_off;
  if (device_ == "cuda") {
    cudaCheck(cudaDeviceSynchronize(), "rebind: draining the device");
    if (auto dev = getDev("cuda")) static_cast<CudaDevice*>(dev.get())->multicastRelease(&mc_);
    mc_base_ = nullptr;
    cudaCheck(cudaMemset(heap_ + layout_.signal_off, 0, ctl), "rebind: clearing the signal area");
    cudaCheck(cudaDeviceSynchronize(), "rebind");
  } else if (heap_) {
    std::memset(heap_ + layout_.signal_off, 0, ctl);
  }
  lane_epochs_.assign(lane_epochs_.size(), 0);
  lane_launches_.assign(lane_launches_.size(), 0);
  for (auto& kv : ops_)
    for (auto& v : kv.second.variants) v.second.epoch = 0;
}

void Engine::injectFault(const std::string& kind) {
  if (!cluster_) throw std::runtime_error("injectFault: not in a cluster");
  if (kind == "silence") cluster_->daemon().injectSilence(true);
  else if (kind == "close") cluster_->daemon().injectAbruptClose();
  else throw std::runtime_error("injectFault: unknown kind (silence|close)");
}

void Engine::regOp(const std::string& name, const std::string& path_or_json) {
  size_t i = path_or_json.find_first_not_of(" \t\r\n");
  Json doc = (i != std::string::npos && path_or_json[i] == '{') ? Json::parse(path_or_json) : Json::parseFile(path_or_json);
  Program p = Program::fromJson(doc);
  PCCL_DLOG_DEBUG("regOp '%s': %s for %d ranks, %d channels, %u signal slots", name.c_str(), p.collective.c_str(), p.world,
                  p.channels, p.num_slots);
  std::lock_guard<std::mutex> g(mu_);
  if (ops_.count(name)) throw std::runtime_error("regOp: '" + name + "' is already registered");
  Op op;
  op.program = std::move(p);
  ops_.emplace(name, std::move(op));
}

uint64_t Engine::heapBase(int rank) const {
  if (rank < 0 || rank >= static_cast<int>(peer_heaps_.size())) return 0;
  return reinterpret_cast<uint64_t>(peer_heaps_[rank]);
}

uint64_t Engine::allocSymmetric(uint64_t bytes, uint64_t align) {
  if (align < 256) align = 256;
  uint64_t off = alignUp(user_top_, align);
  if (off + bytes > layout_.total) throw std::runtime_error("allocSymmetric: symmetric heap exhausted (raise heap_bytes)");
  user_top_ = off + bytes;
  return off;
}

void Engine::resetSymmetric(uint64_t mark) {
  if (mark < layout_.user_off || mark > layout_.total) throw std::runtime_error("resetSymmetric: bad mark");
  user_top_ = mark;
}

World Engine::worldTable() const {
  if (mixed_hosts_)
    throw std::runtime_error("this kernel addresses every peer's memory directly, but the ranks of this world span several hosts "
                             "(use a program through exeOp: it runs on the host-driven executor)");
  World w{};
  w.world = world_;
  for (int r = 0; r < world_; ++r) w.heap[r] = peer_heaps_[r];
  w.mc_heap = static_cast<char*>(mc_base_);
  w.signal_off = layout_.signal_off;
  w.flag_off = layout_.flag_off;
  return w;
}

bool Engine::multicastSupported() {
  if (device_ != "cuda") return false;
  return static_cast<CudaDevice*>(getDev("cuda").get())->multicastSupported();
}

std::string Engine::mcCreate() {
  auto* dev = static_cast<CudaDevice*>(getDev("cuda").get());
  size_t gran = dev->multicastGranularity(world_, layout_.total);
  if (layout_.total % gran) throw std::runtime_error("mcCreate: heap size is not a multiple of the multicast granularity");
  return dev->multicastCreate(layout_.total, world_, &mc_);
}

void Engine::mcJoin(const std::string& handle) { static_cast<CudaDevice*>(getDev("cuda").get())->multicastJoin(handle, &mc_); }

void Engine::mcBind() { mc_base_ = static_cast<CudaDevice*>(getDev("cuda").get())->multicastBind(heap_, &mc_); }

uint64_t Engine::nextEpoch(int lane) {
  if (lane < 0 || lane >= static_cast<int>(lane_epochs_.size())) throw std::runtime_error("nextEpoch: bad lane");
  return ++lane_epochs_[lane];
}

uint64_t Engine::statusPtr(int lane) const { return reinterpret_cast<uint64_t>(heap_ + layout_.status_off + 64ull * lane); }

std::vector<uint32_t> Engine::checkStatus(int lane) {
  std::vector<uint32_t> st(4, 0);
  if (device_ == "cuda") {
    cudaCheck(cudaDeviceSynchronize(), "checkStatus");
    cudaCheck(cudaMemcpy(st.data(), reinterpret_cast<void*>(statusPtr(lane)), 16, cudaMemcpyDeviceToHost), "reading status");
    if (st[0] != ST_OK) cudaMemset(reinterpret_cast<void*>(statusPtr(lane)), 0, 16);
  } else {
    std::memcpy(st.data(), reinterpret_cast<void*>(statusPtr(lane)), 16);
    std::memset(reinterpret_cast<void*>(statusPtr(lane)), 0, 16);
  }
  return st;
}

int Engine::exeOp(const std::string& name, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes,
                  const std::string& dtype, int width, int lane, uint64_t stream) {
  if (!initialized_) throw std::runtime_error("exeOp: call initEngine first");
  PCCL_DLOG_TRACE("exeOp '%s': %llu bytes of %s, width %d, lane %d", name.c_str(), static_cast<unsigned long long>(in_bytes),
                  dtype.c_str(), width, lane);
  Op* found = nullptr;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = ops_.find(name);
    if (it == ops_.end()) throw std::runtime_error("exeOp: no op named '" + name + "'");
    found = &it->second;                 // std::map nodes are stable; ops are never unregistered
  }
  Op& op = *found;
  if (op.program.world != world_) throw std::runtime_error("exeOp: '" + name + "' was written for another world size");
  if (lane < 0 || lane >= layout_.lanes) throw std::runtime_error("exeOp: lane out of range");
  for (int r = 0; r < world_; ++r)
    if (r != rank_ && !peer_heaps_[r] && !(tcp_ && (device_ == "cpu" || mixed_hosts_)))
      throw std::runtime_error("exeOp: peers are not connected (joinCluster/importEndpoints first)");
  uint32_t dt = parseDType(dtype);
  if (width < 1) width = 1;
  if (width > max_width_) width = max_width_;
  if (device_ == "cpu") return exeOnCpu(op, in_ptr, out_ptr, in_bytes, dt, width, lane);
  if (mixed_hosts_) return exeOnCudaHost(op, in_ptr, out_ptr, in_bytes, dt, width, lane, stream);
  return exeOnCuda(op, in_ptr, out_ptr, in_bytes, dt, width, lane, stream);
}

// Signal words of a (program, width) pair are handed out at its first launch; every rank launches the same sequence
// of (op, width) pairs, so every rank arrives at the same numbering.
void Engine::prepareOp(const std::string& name, int width) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = ops_.find(name);
  if (it == ops_.end()) throw std::runtime_error("prepareOp: no op named '" + name + "'");
  if (width < 1) width = 1;
  if (width > max_width_) width = max_width_;
  variantFor(it->second, width);
}

// (callers hold mu_)
Engine::Op::Variant& Engine::variantFor(Op& op, int width) {
  auto it = op.variants.find(width);
  if (it != op.variants.end()) return it->second;
  const uint32_t need = op.program.num_slots * static_cast<uint32_t>(width);
  if (next_slot_ + need > layout_.turn_base) throw std::runtime_error("exeOp: out of signal words");
  Op::Variant v;
  v.slot_base = next_slot_;
  next_slot_ += need;
  return op.variants.emplace(width, v).first->second;
}

int Engine::exeOnCpu(Op& op, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, uint32_t dt, int width, int lane) {
  const Program& p = op.program;
  uint64_t bb = p.blockBytesForInput(in_bytes);
  if (bb % dtypeSize(dt)) throw std::runtime_error("exeOp: block size is not a whole number of elements");
  if (p.needs_multicast || p.remote_io) throw std::runtime_error("exeOp: this program needs GPU symmetric memory");
  auto key = std::make_pair(bb, width);
  std::unique_lock<std::mutex> lock(mu_);      // bookkeeping is serialised; the execution itself is not
  auto hc = op.host_cache.find(key);
  if (hc == op.host_cache.end()) hc = op.host_cache.emplace(key, p.materialize(rank_, bb, width)).first;
  const Materialized& m = hc->second;
  uint64_t lane_bytes = layout_.workspace_bytes / layout_.lanes, half = lane_bytes / 2 / 4096 * 4096;
  if (m.buf_bytes[BUF_SCRATCH] > half)
    throw std::runtime_error("exeOp: message needs " + std::to_string(m.buf_bytes[BUF_SCRATCH]) +
                             " bytes of scratch but a workspace lane half holds " + std::to_string(half) +
                             " (raise PCCL_WORKSPACE_MB or split the message)");
  Op::Variant& var = variantFor(op, width);
  const uint64_t launch_no = lane_launches_.at(lane)++;
  uint64_t scratch_off = lane * lane_bytes + (launch_no & 1) * half;
  CpuExecContext ctx;
  ctx.turn_slot = world_ > 1 ? static_cast<int64_t>(layout_.turn_base) + lane * kMaxRanks : -1;
  ctx.launch_no = launch_no;
  if (exec_delay_rank_ == rank_) ctx.delay_us = exec_delay_us_;
  ctx.rank = rank_;
  ctx.world = world_;
  ctx.local[BUF_INPUT] = reinterpret_cast<char*>(in_ptr);
  ctx.local[BUF_OUTPUT] = reinterpret_cast<char*>(p.in_place ? in_ptr : out_ptr);
  ctx.local[BUF_SCRATCH] = heap_ + scratch_off;
  for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b) ctx.local_bytes[b] = m.buf_bytes[b];
  ctx.peer_scratch.assign(world_, nullptr);
  ctx.peer_signals.assign(world_, nullptr);
  for (int r = 0; r < world_; ++r) {
    if (!peer_heaps_[r]) continue;
    ctx.peer_scratch[r] = peer_heaps_[r] + scratch_off;
    ctx.peer_signals[r] = reinterpret_cast<std::atomic<uint64_t>*>(peer_heaps_[r] + layout_.signal_off);
  }
  ctx.tcp = remote_;
  ctx.tcp_scratch_key = remote_key_;
  ctx.tcp_scratch_off = scratch_off;
  ctx.slot_base = var.slot_base;
  ctx.epoch = var.epoch++;
  ctx.dtype = dt;
  ctx.redop = parseRedOp(p.redop);
  ctx.timeout_ms = timeout_ms_;
  ctx.bounds_check = bounds_check_;
  ctx.trace = trace_;
  lock.unlock();
  CpuExecResult res = runOnCpu(m, ctx);
  lock.lock();
  for (auto& ev : res.trace) spans_.push_back(Span{p.name, ev.stream, ev.pc, ev.op, ev.t0_ns, ev.t1_ns, ev.bytes});
  op.launches++;
  op.bytes += m.bytes_moved;
  op.nanos += res.nanos;
  uint32_t* st = reinterpret_cast<uint32_t*>(statusPtr(lane));
  st[0] = res.status;
  st[1] = static_cast<uint32_t>(res.failed_stream);
  st[2] = static_cast<uint32_t>(res.failed_pc);
  if (res.status == ST_TIMEOUT) op.timeouts++;
  if (res.status != ST_OK)
    PCCL_LOG_ERROR("exeOp '%s': status %u at stream %d pc %d", p.name.c_str(), res.status, res.failed_stream, res.failed_pc);
  return static_cast<int>(res.status);
}

// CUDA engine whose peers are partly on other hosts: the same materialised streams as the CPU executor runs, walked by
// host threads; COPY and REDUCE act on device memory (peers of this host through their NVLink mapping), a COPY to a
// peer on another host goes device -> host -> TCP -> the peer's host shadow -> the peer's device, NOTIFY / WAIT use
// host signal words fed by TCP.  Synchronous: the inputs are awaited on `stream`, the outputs are complete on return.
int Engine::exeOnCudaHost(Op& op, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, uint32_t dt, int width, int lane,
                          uint64_t stream) {
  const Program& p = op.program;
  uint64_t bb = p.blockBytesForInput(in_bytes);
  if (bb % dtypeSize(dt)) throw std::runtime_error("exeOp: block size is not a whole number of elements");
  if (p.needs_multicast || p.remote_io)
    throw std::runtime_error("exeOp: this program needs every rank on one NVSwitch; the ranks of this world span several hosts");
  cudaCheck(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)), "waiting for the inputs");
  auto key = std::make_pair(bb, width);
  std::unique_lock<std::mutex> lock(mu_);
  auto hc = op.host_cache.find(key);
  if (hc == op.host_cache.end()) hc = op.host_cache.emplace(key, p.materialize(rank_, bb, width)).first;
  const Materialized& m = hc->second;
  uint64_t lane_bytes = layout_.workspace_bytes / layout_.lanes, half = lane_bytes / 2 / 4096 * 4096;
  if (m.buf_bytes[BUF_SCRATCH] > half) throw std::runtime_error("exeOp: message needs more scratch than a workspace lane half holds (raise PCCL_WORKSPACE_MB)");
  Op::Variant& var = variantFor(op, width);
  const uint64_t launch_no = lane_launches_.at(lane)++;
  uint64_t scratch_off = lane * lane_bytes + (launch_no & 1) * half;
  CpuExecContext ctx;
  ctx.turn_slot = static_cast<int64_t>(layout_.turn_base) + lane * kMaxRanks;
  ctx.launch_no = launch_no;
  ctx.rank = rank_;
  ctx.world = world_;
  ctx.local[BUF_INPUT] = reinterpret_cast<char*>(in_ptr);
  ctx.local[BUF_OUTPUT] = reinterpret_cast<char*>(p.in_place ? in_ptr : out_ptr);
  ctx.local[BUF_SCRATCH] = heap_ + scratch_off;
  for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b) ctx.local_bytes[b] = m.buf_bytes[b];
  ctx.peer_scratch.assign(world_, nullptr);
  ctx.peer_signals.assign(world_, nullptr);
  for (int r = 0; r < world_; ++r)
    if (peer_heaps_[r]) ctx.peer_scratch[r] = peer_heaps_[r] + scratch_off;
  ctx.peer_signals[rank_] = host_signals_;
  ctx.tcp = tcp_.get();
  ctx.tcp_scratch_key = tcp_key_;
  ctx.tcp_scratch_off = scratch_off;
  ctx.slot_base = var.slot_base;
  ctx.epoch = var.epoch++;
  ctx.dtype = dt;
  ctx.redop = parseRedOp(p.redop);
  ctx.timeout_ms = timeout_ms_;
  ctx.bounds_check = bounds_check_;
  ctx.mem = device_mem_ops_.get();
  lock.unlock();
  CpuExecResult res = runOnCpu(m, ctx);
  lock.lock();
  op.launches++;
  op.bytes += m.bytes_moved;
  op.nanos += res.nanos;
  if (res.status == ST_TIMEOUT) op.timeouts++;
  if (res.status != ST_OK) {
    uint32_t st[4] = {res.status, static_cast<uint32_t>(res.failed_stream), static_cast<uint32_t>(res.failed_pc), 0};
    cudaMemcpy(reinterpret_cast<void*>(statusPtr(lane)), st, sizeof(st), cudaMemcpyHostToDevice);
    PCCL_LOG_ERROR("exeOp '%s' (host-driven): status %u at stream %d pc %d", p.name.c_str(), res.status, res.failed_stream, res.failed_pc);
  }
  return static_cast<int>(res.status);
}

int Engine::exeOnCuda(Op& op, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, uint32_t dt, int width, int lane,
                      uint64_t stream) {
  const Program& p = op.program;
  uint64_t bb = p.blockBytesForInput(in_bytes);
  if (bb % dtypeSize(dt)) throw std::runtime_error("exeOp: block size is not a whole number of elements");
  if (p.needs_multicast && !mc_base_) throw std::runtime_error("exeOp: program needs NVLS multicast, which is not set up");
  auto key = std::make_pair(bb, width);
  std::unique_lock<std::mutex> lock(mu_);      // the launch is asynchronous, so the whole call may hold the lock
  auto dc = op.device_cache.find(key);
  if (dc == op.device_cache.end()) {
    Op::DeviceCopy c;
    c.m = p.materialize(rank_, bb, width);
    std::vector<Instr> flat;
    std::vector<uint32_t> starts;
    for (auto& s : c.m.streams) {
      starts.push_back(static_cast<uint32_t>(flat.size()));
      flat.insert(flat.end(), s.begin(), s.end());
    }
    c.n_streams = static_cast<int>(starts.size());
    flat.resize(flat.size() + kInstrPad, Instr{});      // the kernel reads whole chunks: no-ops behind the last stream
    cudaCheck(cudaMalloc(&c.instrs, flat.size() * sizeof(Instr)), "cudaMalloc(instructions)");
    cudaCheck(cudaMalloc(&c.starts, starts.size() * sizeof(uint32_t)), "cudaMalloc(stream table)");
    cudaCheck(cudaMemcpy(c.instrs, flat.data(), flat.size() * sizeof(Instr), cudaMemcpyHostToDevice), "upload instructions");
    cudaCheck(cudaMemcpy(c.starts, starts.data(), starts.size() * sizeof(uint32_t), cudaMemcpyHostToDevice), "upload stream table");
    dc = op.device_cache.emplace(key, std::move(c)).first;
  }
  const Op::DeviceCopy& c = dc->second;
  uint64_t lane_bytes = layout_.workspace_bytes / layout_.lanes, half = lane_bytes / 2 / 4096 * 4096;
  if (c.m.buf_bytes[BUF_SCRATCH] > half)
    throw std::runtime_error("exeOp: message needs more scratch than a workspace lane half holds (raise PCCL_WORKSPACE_MB)");
  auto heapOff = [&](uint64_t ptr) -> long long {
    uint64_t base = reinterpret_cast<uint64_t>(heap_);
    return (ptr >= base && ptr < base + layout_.total) ? static_cast<long long>(ptr - base) : -1;
  };
  InterpLaunch L{};
  L.w = worldTable();
  L.nvirt = 1;
  Op::Variant& var = variantFor(op, width);
  L.slot_base = var.slot_base;
  L.epoch = var.epoch;
  L.dtype = dt;
  L.redop = parseRedOp(p.redop);
  L.spin_limit = spin_limit_;
  L.bounds_check = bounds_check_ ? 1 : 0;
  InterpRank& R = L.r[0];
  R.rank = rank_;
  R.n_streams = c.n_streams;
  R.instrs = c.instrs;
  R.stream_start = c.starts;
  R.input = reinterpret_cast<char*>(in_ptr);
  R.output = reinterpret_cast<char*>(p.in_place ? in_ptr : out_ptr);
  R.input_heap_off = heapOff(in_ptr);
  R.output_heap_off = heapOff(p.in_place ? in_ptr : out_ptr);
  if (p.remote_io && (R.input_heap_off < 0 || R.output_heap_off < 0))
    throw std::runtime_error("exeOp: this program lets peers touch the tensors, so both must come from the symmetric heap");
  const uint64_t launch_no = lane_launches_.at(lane)++;
  R.scratch_off = lane * lane_bytes + (launch_no & 1) * half;
  if (world_ > 1) {
    L.turn_slot = layout_.turn_base + static_cast<uint32_t>(lane) * kMaxRanks;
    L.finish_slot = layout_.finish_base + static_cast<uint32_t>(lane);
    L.launch_no = launch_no;
  }
  for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b) R.buf_bytes[b] = c.m.buf_bytes[b];
  R.status = reinterpret_cast<uint32_t*>(statusPtr(lane));
  size_t n_instr = 0;
  if (trace_) {
    for (auto& s : c.m.streams) n_instr += s.size();
    if (dtrace_.size() <= static_cast<size_t>(lane)) dtrace_.resize(lane + 1);
    DeviceTrace& t = dtrace_[lane];
    if (t.cap < 2 * n_instr) {
      if (t.words) cudaFree(t.words);
      t.words = nullptr;
      t.cap = 0;
      cudaCheck(cudaMalloc(&t.words, 2 * n_instr * sizeof(uint64_t)), "cudaMalloc(trace)");
      t.cap = 2 * n_instr;
    }
    cudaCheck(cudaMemsetAsync(t.words, 0, 2 * n_instr * sizeof(uint64_t), reinterpret_cast<cudaStream_t>(stream)), "clearing the trace");
    R.trace = t.words;
  }
  int err = launchInterpreter(L, 512, reinterpret_cast<cudaStream_t>(stream));
  if (err != 0) throw std::runtime_error(std::string("exeOp: kernel launch failed: ") + cudaErrorName(err));
  var.epoch++;
  op.launches++;
  op.bytes += c.m.bytes_moved;
  if (trace_) {
    // Read the stamps back without the lock: the kernel may be waiting for a peer whose matching launch
    // on another lane of this engine needs the lock first.
    uint64_t* words = R.trace;
    lock.unlock();
    cudaCheck(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)), "traced launch");
    std::vector<uint64_t> stamps(2 * n_instr);
    cudaCheck(cudaMemcpy(stamps.data(), words, stamps.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost), "reading the trace");
    lock.lock();
    addDeviceSpans(p.name, c.m, stamps);
  }
  return 0;
}

// ---- hooks for run-time compiled kernels ----------------------------------------------------------------------------
std::vector<std::vector<Instr>> Engine::materializedStreams(const std::string& name, uint64_t in_bytes, int width, uint64_t* buf_bytes) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = ops_.find(name);
  if (it == ops_.end()) throw std::runtime_error("materializedStreams: no op named '" + name + "'");
  const Program& p = it->second.program;
  if (width < 1) width = 1;
  if (width > max_width_) width = max_width_;
  Materialized m = p.materialize(rank_, p.blockBytesForInput(in_bytes), width);
  if (buf_bytes)
    for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b) buf_bytes[b] = m.buf_bytes[b];
  return m.streams;
}

std::map<std::string, std::string> Engine::opInfo(const std::string& name) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = ops_.find(name);
  if (it == ops_.end()) throw std::runtime_error("opInfo: no op named '" + name + "'");
  const Program& p = it->second.program;
  return {{"name", p.name}, {"collective", p.collective}, {"redop", p.redop}, {"world", std::to_string(p.world)},
          {"channels", std::to_string(p.channels)}, {"in_place", p.in_place ? "1" : "0"}, {"needs_multicast", p.needs_multicast ? "1" : "0"},
          {"remote_io", p.remote_io ? "1" : "0"}};
}

Engine::LaunchPlan Engine::planLaunch(const std::string& name, uint64_t in_bytes, int width, int lane) {
  if (!initialized_ || device_ != "cuda") throw std::runtime_error("planLaunch: a CUDA engine is needed");
  if (mixed_hosts_) throw std::runtime_error("planLaunch: the ranks of this world span several hosts");
  std::lock_guard<std::mutex> g(mu_);
  auto it = ops_.find(name);
  if (it == ops_.end()) throw std::runtime_error("planLaunch: no op named '" + name + "'");
  Op& op = it->second;
  if (op.program.world != world_) throw std::runtime_error("planLaunch: '" + name + "' was written for another world size");
  if (lane < 0 || lane >= layout_.lanes) throw std::runtime_error("planLaunch: lane out of range");
  if (op.program.needs_multicast && !mc_base_) throw std::runtime_error("planLaunch: program needs NVLS multicast, which is not set up");
  if (width < 1) width = 1;
  if (width > max_width_) width = max_width_;
  for (int r = 0; r < world_; ++r)
    if (r != rank_ && !peer_heaps_[r]) throw std::runtime_error("planLaunch: peers are not connected");
  Materialized m = op.program.materialize(rank_, op.program.blockBytesForInput(in_bytes), width);
  uint64_t lane_bytes = layout_.workspace_bytes / layout_.lanes, half = lane_bytes / 2 / 4096 * 4096;
  if (m.buf_bytes[BUF_SCRATCH] > half) throw std::runtime_error("planLaunch: message needs more scratch than a workspace lane half holds");
  Op::Variant& var = variantFor(op, width);
  LaunchPlan L{};
  L.slot_base = var.slot_base;
  L.epoch = var.epoch++;
  L.launch_no = lane_launches_.at(lane)++;
  L.scratch_off = lane * lane_bytes + (L.launch_no & 1) * half;
  L.turn_slot = world_ > 1 ? layout_.turn_base + static_cast<uint32_t>(lane) * kMaxRanks : kNoTurnSlot;
  L.finish_slot = layout_.finish_base + static_cast<uint32_t>(lane);
  L.spin_limit = spin_limit_;
  L.status_ptr = statusPtr(lane);
  L.signal_off = layout_.signal_off;
  L.mc_base = reinterpret_cast<uint64_t>(mc_base_);
  op.launches++;
  op.bytes += m.bytes_moved;
  return L;
}

// ---- resident executor ---------------------------------------------------------------------------------------------
void Engine::startResident(int width) {
  if (!initialized_ || device_ != "cuda") throw std::runtime_error("startResident: a CUDA engine is needed");
  if (mixed_hosts_) throw std::runtime_error("startResident: the ranks of this world span several hosts");
  std::lock_guard<std::mutex> g(mu_);
  if (rq_host_) throw std::runtime_error("startResident: already started");
  if (width < 1) width = 1;
  if (width > max_width_) width = max_width_;
  void* hp = nullptr;
  cudaCheck(cudaHostAlloc(&hp, sizeof(ResidentQueue), cudaHostAllocMapped), "resident queue");
  std::memset(hp, 0, sizeof(ResidentQueue));
  rq_host_ = static_cast<ResidentQueue*>(hp);
  void* dp = nullptr;
  cudaCheck(cudaHostGetDevicePointer(&dp, hp, 0), "resident queue (device view)");
  rq_dev_ = static_cast<ResidentQueue*>(dp);
  rq_host_->idle_ns = static_cast<uint64_t>(LaunchEnvironments::getInt("PCCL_RESIDENT_IDLE_MS", 20)) * 1000000ull;
  cudaCheck(cudaMalloc(reinterpret_cast<void**>(&rctl_), sizeof(ResidentCtl)), "resident control block");
  cudaCheck(cudaMemset(rctl_, 0, sizeof(ResidentCtl)), "resident control block");
  cudaStream_t s = nullptr;
  cudaCheck(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "resident stream");
  resident_stream_ = s;
  resident_width_ = width;
  launchResidentKernel();
}

void Engine::launchResidentKernel() {
  cudaStream_t s = static_cast<cudaStream_t>(resident_stream_);
  cudaCheck(cudaStreamSynchronize(s), "resident kernel (previous run)");       // it has left: running == 0
  rq_host_->stop = 0;
  rq_host_->running = 1;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  // every program of a launch may have up to width x channels streams; the grid must hold the widest registered one,
  // which is checked per enqueue -- here the grid is sized for the budget
  int err = launchResident(rq_dev_, rctl_, rq_host_->completed, resident_width_ * kResidentChannels, 512, s);
  if (err != 0) {
    rq_host_->running = 0;
    throw std::runtime_error(std::string("startResident: kernel launch failed: ") + cudaErrorName(err));
  }
  resident_launches_++;
}

uint64_t Engine::enqueueOp(const std::string& name, uint64_t in_ptr, uint64_t out_ptr, uint64_t in_bytes, const std::string& dtype, int lane,
                           uint64_t stream) {
  if (!rq_host_) throw std::runtime_error("enqueueOp: call startResident first");
  if (stream) cudaCheck(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)), "enqueueOp: waiting for the inputs");
  std::unique_lock<std::mutex> lock(mu_);
  auto it = ops_.find(name);
  if (it == ops_.end()) throw std::runtime_error("enqueueOp: no op named '" + name + "'");
  Op& op = it->second;
  const Program& p = op.program;
  if (p.world != world_) throw std::runtime_error("enqueueOp: '" + name + "' was written for another world size");
  if (lane < 0 || lane >= layout_.lanes) throw std::runtime_error("enqueueOp: lane out of range");
  const int width = resident_width_;
  const uint32_t dt = parseDType(dtype);
  uint64_t bb = p.blockBytesForInput(in_bytes);
  if (bb % dtypeSize(dt)) throw std::runtime_error("enqueueOp: block size is not a whole number of elements");
  if (p.needs_multicast && !mc_base_) throw std::runtime_error("enqueueOp: program needs NVLS multicast, which is not set up");
  auto key = std::make_pair(bb, width);
  auto dc = op.device_cache.find(key);
  if (dc == op.device_cache.end()) {
    Op::DeviceCopy c;
    c.m = p.materialize(rank_, bb, width);
    std::vector<Instr> flat;
    std::vector<uint32_t> starts;
    for (auto& st : c.m.streams) {
      starts.push_back(static_cast<uint32_t>(flat.size()));
      flat.insert(flat.end(), st.begin(), st.end());
    }
    c.n_streams = static_cast<int>(starts.size());
    flat.resize(flat.size() + kInstrPad, Instr{});
    cudaCheck(cudaMalloc(&c.instrs, flat.size() * sizeof(Instr)), "cudaMalloc(instructions)");
    cudaCheck(cudaMalloc(&c.starts, (starts.size() + 1) * sizeof(uint32_t)), "cudaMalloc(stream table)");
    cudaCheck(cudaMemcpy(c.instrs, flat.data(), flat.size() * sizeof(Instr), cudaMemcpyHostToDevice), "upload instructions");
    if (!starts.empty()) cudaCheck(cudaMemcpy(c.starts, starts.data(), starts.size() * sizeof(uint32_t), cudaMemcpyHostToDevice), "upload stream table");
    dc = op.device_cache.emplace(key, std::move(c)).first;
  }
  const Op::DeviceCopy& c = dc->second;
  if (c.n_streams > resident_width_ * kResidentChannels)
    throw std::runtime_error("enqueueOp: '" + name + "' has more streams than the resident kernel has CTAs (fewer channels, or a wider kernel)");
  uint64_t lane_bytes = layout_.workspace_bytes / layout_.lanes, half = lane_bytes / 2 / 4096 * 4096;
  if (c.m.buf_bytes[BUF_SCRATCH] > half) throw std::runtime_error("enqueueOp: message needs more scratch than a workspace lane half holds");
  // room in the ring
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms_);
  while (rq_host_->tail - rq_host_->completed >= kResidentSlots) {
    if (std::chrono::steady_clock::now() >= deadline) throw std::runtime_error("enqueueOp: the resident queue stayed full");
    std::this_thread::yield();
  }
  auto heapOff = [&](uint64_t ptr) -> long long {
    uint64_t base = reinterpret_cast<uint64_t>(heap_);
    return (ptr >= base && ptr < base + layout_.total) ? static_cast<long long>(ptr - base) : -1;
  };
  ResidentDesc d{};
  d.w = worldTable();
  Op::Variant& var = variantFor(op, width);
  d.slot_base = var.slot_base;
  d.epoch = var.epoch++;
  d.dtype = dt;
  d.redop = parseRedOp(p.redop);
  d.spin_limit = spin_limit_;
  d.bounds_check = bounds_check_ ? 1 : 0;
  d.r.rank = rank_;
  d.r.n_streams = c.n_streams;
  d.r.instrs = c.instrs;
  d.r.stream_start = c.starts;
  d.r.input = reinterpret_cast<char*>(in_ptr);
  d.r.output = reinterpret_cast<char*>(p.in_place ? in_ptr : out_ptr);
  d.r.input_heap_off = heapOff(in_ptr);
  d.r.output_heap_off = heapOff(p.in_place ? in_ptr : out_ptr);
  if (p.remote_io && (d.r.input_heap_off < 0 || d.r.output_heap_off < 0))
    throw std::runtime_error("enqueueOp: this program lets peers touch the tensors, so both must come from the symmetric heap");
  const uint64_t launch_no = lane_launches_.at(lane)++;
  d.r.scratch_off = lane * lane_bytes + (launch_no & 1) * half;
  for (int b = 0; b < static_cast<int>(BUF_COUNT); ++b) d.r.buf_bytes[b] = c.m.buf_bytes[b];
  d.r.status = reinterpret_cast<uint32_t*>(statusPtr(lane));
  d.r.trace = nullptr;
  d.turn_slot = kNoTurnSlot;
  if (world_ > 1) {
    d.turn_slot = layout_.turn_base + static_cast<uint32_t>(lane) * kMaxRanks;
    d.finish_slot = layout_.finish_base + static_cast<uint32_t>(lane);
    d.launch_no = launch_no;
  }
  const uint64_t ticket = rq_host_->tail + 1;
  std::memcpy(const_cast<ResidentDesc*>(&rq_host_->slots[rq_host_->tail % kResidentSlots]), &d, sizeof(d));
  std::atomic_thread_fence(std::memory_order_release);
  rq_host_->tail = ticket;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  // the kernel may have left for lack of work (before or just after this write): start it again; a kernel that is
  // still there simply finds the descriptor
  if (rq_host_->running == 0) launchResidentKernel();
  op.launches++;
  op.bytes += c.m.bytes_moved;
  resident_ops_++;
  return ticket;
}

bool Engine::waitOp(uint64_t ticket, int timeout_ms) {
  if (!rq_host_) throw std::runtime_error("waitOp: the resident executor is not running");
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : timeout_ms_);
  for (int spins = 0; rq_host_->completed < ticket; ++spins) {
    if ((spins & 255) == 255) {
      if (rq_host_->running == 0 && rq_host_->completed < ticket && rq_host_->tail >= ticket) {
        std::lock_guard<std::mutex> g(mu_);
        if (rq_host_->running == 0 && rq_host_->completed < ticket) launchResidentKernel();     // it left between our write and its last look
      }
      if (std::chrono::steady_clock::now() >= deadline) return false;
    }
  }
  std::atomic_thread_fence(std::memory_order_acquire);
  return true;
}

void Engine::stopResident() {
  std::lock_guard<std::mutex> g(mu_);
  if (!rq_host_) return;
  rq_host_->stop = 1;
  std::atomic_thread_fence(std::memory_order_seq_cst);
  cudaStreamSynchronize(static_cast<cudaStream_t>(resident_stream_));
  cudaStreamDestroy(static_cast<cudaStream_t>(resident_stream_));
  resident_stream_ = nullptr;
  cudaFree(rctl_);
  rctl_ = nullptr;
  cudaFreeHost(rq_host_);
  rq_host_ = rq_dev_ = nullptr;
  resident_width_ = 0;
}

void Engine::addDeviceSpans(const std::string& name, const Materialized& m, const std::vector<uint64_t>& stamps) {
  size_t flat = 0;
  for (size_t s = 0; s < m.streams.size(); ++s)
    for (size_t pc = 0; pc < m.streams[s].size(); ++pc, ++flat) {
      const Instr& in = m.streams[s][pc];
      if (2 * flat + 1 >= stamps.size()) return;
      uint64_t t0 = stamps[2 * flat], t1 = stamps[2 * flat + 1];
      if (in.op == OP_END || t0 == 0 || t1 < t0) continue;      // never reached (a failed stream stops early)
      bool moves = in.op == OP_COPY || in.op == OP_REDUCE || in.op == OP_MM_LD_REDUCE || in.op == OP_MM_ST;
      spans_.push_back(Span{name, static_cast<uint32_t>(s), static_cast<uint32_t>(pc), in.op, t0, t1, moves ? in.bytes : 0});
    }
}

void Engine::ingestDeviceTrace(const std::string& name, uint64_t in_bytes, int width, const std::vector<uint64_t>& stamps) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = ops_.find(name);
  if (it == ops_.end()) throw std::runtime_error("ingestDeviceTrace: no operator named '" + name + "'");
  const Program& p = it->second.program;
  Materialized m = p.materialize(rank_, p.blockBytesForInput(in_bytes), width);
  size_t n = 0;
  for (auto& s : m.streams) n += s.size();
  if (stamps.size() != 2 * n)
    throw std::runtime_error("ingestDeviceTrace: " + std::to_string(stamps.size()) + " stamps for " + std::to_string(n) + " instructions");
  addDeviceSpans(name, m, stamps);
}

std::string Engine::trace() {
  std::lock_guard<std::mutex> lock(mu_);
  static const char* names[] = {"NOP", "COPY", "REDUCE", "NOTIFY", "WAIT", "MM_LD_REDUCE", "MM_ST", "BARRIER", "END"};
  Json events = Json::array();
  for (auto& s : spans_) {
    Json e = Json::object();
    e.set("name", std::string(names[s.opcode < 9 ? s.opcode : 0]));
    e.set("cat", s.op);
    e.set("ph", "X");
    e.set("pid", rank_);
    e.set("tid", static_cast<int64_t>(s.stream));
    e.set("ts", static_cast<double>(s.t0) / 1000.0);
    e.set("dur", static_cast<double>(s.t1 - s.t0) / 1000.0);
    Json args = Json::object();
    args.set("pc", static_cast<int64_t>(s.pc));
    args.set("bytes", s.bytes);
    e.set("args", args);
    events.push(e);
  }
  spans_.clear();
  Json doc = Json::object();
  doc.set("traceEvents", events);
  doc.set("displayTimeUnit", "ns");
  return doc.dump();
}

std::string Engine::stats() {
  Json j = Json::object();
  j.set("rank", rank_);
  j.set("world", world_);
  j.set("device", device_);
  j.set("heap_bytes", layout_.total);
  j.set("workspace_bytes", layout_.workspace_bytes);
  j.set("signals_used", static_cast<uint64_t>(next_slot_));
  j.set("multicast", mc_base_ != nullptr);
  j.set("mixed_hosts", mixed_hosts_);
  j.set("resident_width", resident_width_);
  j.set("resident_kernel_launches", resident_launches_);
  j.set("resident_ops", resident_ops_);
  j.set("log_file", Logger::get().path());
  j.set("log_errors", Logger::get().count(LogLevel::Error));
  if (verbs_) {
    j.set("verbs_bytes_sent", verbs_->bytesSent());
    for (int r = 0; r < world_; ++r)
      if (r != rank_) j.set("verbs_qp_state." + std::to_string(r), verbs_->queuePairState(r));
  }
  if (tcp_) {
    j.set("tcp_bytes_sent", tcp_->bytesSent());
    j.set("tcp_bytes_received", tcp_->bytesReceived());
  }
  Json ops = Json::object();
  for (auto& kv : ops_) {
    Json o = Json::object();
    o.set("collective", kv.second.program.collective);
    o.set("launches", kv.second.launches);
    o.set("bytes", kv.second.bytes);
    o.set("timeouts", kv.second.timeouts);
    o.set("host_nanos", kv.second.nanos);
    double gbps = kv.second.nanos ? static_cast<double>(kv.second.bytes) / static_cast<double>(kv.second.nanos) : 0.0;
    o.set("host_gb_per_s", gbps);
    o.set("fingerprint", fnv1a(kv.second.program.name));
    ops.set(kv.first, o);
  }
  j.set("ops", ops);
  return j.dump();
}

}  // namespace pccl
