#include "verbs_transport.h"

#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>

#include "../common/env.h"
#include "../common/hex.h"
#include "../common/json.h"
#include "../common/log.h"
#include "verbs_abi.h"

namespace pccl {

// ---- the library, resolved once per name -----------------------------------------------------------------------
struct VerbsApi {
  void* lib = nullptr;
  std::string why;
  ibv_device** (*get_device_list)(int*) = nullptr;
  void (*free_device_list)(ibv_device**) = nullptr;
  const char* (*get_device_name)(ibv_device*) = nullptr;
  ibv_context* (*open_device)(ibv_device*) = nullptr;
  int (*close_device)(ibv_context*) = nullptr;
  int (*query_port)(ibv_context*, uint8_t, ibv_port_attr*) = nullptr;
  int (*query_gid)(ibv_context*, uint8_t, int, ibv_gid*) = nullptr;
  ibv_pd* (*alloc_pd)(ibv_context*) = nullptr;
  int (*dealloc_pd)(ibv_pd*) = nullptr;
  ibv_mr* (*reg_mr)(ibv_pd*, void*, size_t, int) = nullptr;
  int (*dereg_mr)(ibv_mr*) = nullptr;
  ibv_cq* (*create_cq)(ibv_context*, int, void*, ibv_comp_channel*, int) = nullptr;
  int (*destroy_cq)(ibv_cq*) = nullptr;
  ibv_qp* (*create_qp)(ibv_pd*, ibv_qp_init_attr*) = nullptr;
  int (*modify_qp)(ibv_qp*, ibv_qp_attr*, int) = nullptr;
  int (*destroy_qp)(ibv_qp*) = nullptr;
  bool ok() const { return lib != nullptr && why.empty(); }
  ~VerbsApi() {
    if (lib) ::dlclose(lib);
  }
};

namespace {

std::shared_ptr<VerbsApi> loadApi() {
  static std::mutex mu;
  static std::map<std::string, std::weak_ptr<VerbsApi>> cache;
  const std::string name = LaunchEnvironments::getStr("PCCL_IBVERBS_LIB", "");
  std::lock_guard<std::mutex> g(mu);
  if (auto live = cache[name].lock()) return live;
  auto api = std::make_shared<VerbsApi>();
  if (!name.empty()) api->lib = ::dlopen(name.c_str(), RTLD_NOW | RTLD_LOCAL);
  else {
    api->lib = ::dlopen("libibverbs.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!api->lib) api->lib = ::dlopen("libibverbs.so", RTLD_NOW | RTLD_LOCAL);
  }
  if (!api->lib) {
    api->why = "libibverbs is not installed";
    return api;
  }
  auto need = [&](const char* sym, void** fn) {
    *fn = ::dlsym(api->lib, sym);
    if (!*fn && api->why.empty()) api->why = std::string("libibverbs lacks ") + sym;
  };
#define PCCL_IBV(field, sym) need(sym, reinterpret_cast<void**>(&api->field))
  PCCL_IBV(get_device_list, "ibv_get_device_list");
  PCCL_IBV(free_device_list, "ibv_free_device_list");
  PCCL_IBV(get_device_name, "ibv_get_device_name");
  PCCL_IBV(open_device, "ibv_open_device");
  PCCL_IBV(close_device, "ibv_close_device");
  PCCL_IBV(query_port, "ibv_query_port");
  PCCL_IBV(query_gid, "ibv_query_gid");
  PCCL_IBV(alloc_pd, "ibv_alloc_pd");
  PCCL_IBV(dealloc_pd, "ibv_dealloc_pd");
  PCCL_IBV(reg_mr, "ibv_reg_mr");
  PCCL_IBV(dereg_mr, "ibv_dereg_mr");
  PCCL_IBV(create_cq, "ibv_create_cq");
  PCCL_IBV(destroy_cq, "ibv_destroy_cq");
  PCCL_IBV(create_qp, "ibv_create_qp");
  PCCL_IBV(modify_qp, "ibv_modify_qp");
  PCCL_IBV(destroy_qp, "ibv_destroy_qp");
#undef PCCL_IBV
  cache[name] = api;
  return api;
}

constexpr size_t kBounceBytes = 1 << 20;
const char* stateName(int s) {
  static const char* n[] = {"RESET", "INIT", "RTR", "RTS", "SQD", "SQE", "ERR"};
  return s >= 0 && s < 7 ? n[s] : "?";
}
constexpr int kAccess = IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ | IBV_ACCESS_REMOTE_ATOMIC;

}  // namespace

bool VerbsTransport::probe(std::string* why) {
  if (LaunchEnvironments::has("PCCL_DISABLE_IB")) {
    if (why) *why = "disabled by PCCL_DISABLE_IB";
    return false;
  }
  auto api = loadApi();
  if (!api->ok()) {
    if (why) *why = api->why;
    return false;
  }
  int n = 0;
  ibv_device** list = api->get_device_list(&n);
  if (list) api->free_device_list(list);
  if (n <= 0) {
    if (why) *why = "no verbs device present";
    return false;
  }
  if (why) *why = std::to_string(n) + " verbs device(s) present";
  return true;
}

VerbsTransport::VerbsTransport(int rank, int world) : rank_(rank), world_(world) {
  if (world < 1 || rank < 0 || rank >= world) throw std::runtime_error("verbs transport: need 0 <= rank < world");
  timeout_ms_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_WAIT_TIMEOUT_MS", 30000));
}

VerbsTransport::~VerbsTransport() { shutdown(); }

bool VerbsTransport::remoteCommAvailable() {
  std::string why;
  return probe(&why);
}

std::string VerbsTransport::activate() {
  std::lock_guard<std::mutex> g(mu_);
  if (active_) return endpoint();
  api_ = loadApi();
  if (!api_->ok()) throw std::runtime_error("verbs transport: " + api_->why);
  // the reference reads these with stoi and throws when they are unset (rdma_executor/device.cc:46-50); here they default
  port_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_IB_PORT_NUM", 1));
  gid_index_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_IB_GID_INDEX", 0));
  const std::string want = LaunchEnvironments::getStr("PCCL_IB_DEVICE", "");
  int n = 0;
  ibv_device** list = api_->get_device_list(&n);
  if (!list || n <= 0) throw std::runtime_error("verbs transport: no verbs device present");
  ibv_device* dev = nullptr;
  for (int i = 0; i < n && !dev; ++i)
    if (want.empty() || want == api_->get_device_name(list[i])) dev = list[i];
  ibv_context* ctx = dev ? api_->open_device(dev) : nullptr;
  api_->free_device_list(list);
  if (!ctx) throw std::runtime_error("verbs transport: cannot open device '" + want + "'");
  ctx_ = ctx;
  ibv_port_attr pa;
  std::memset(&pa, 0, sizeof(pa));
  if (api_->query_port(ctx, static_cast<uint8_t>(port_), &pa) != 0) throw std::runtime_error("verbs transport: ibv_query_port failed");
  lid_ = pa.lid;
  ibv_gid gid;
  std::memset(&gid, 0, sizeof(gid));
  if (api_->query_gid(ctx, static_cast<uint8_t>(port_), gid_index_, &gid) != 0) throw std::runtime_error("verbs transport: ibv_query_gid failed");
  std::memcpy(gid_, gid.raw, 16);
  pd_ = api_->alloc_pd(ctx);
  if (!pd_) throw std::runtime_error("verbs transport: ibv_alloc_pd failed");
  cq_ = api_->create_cq(ctx, 4096, nullptr, nullptr, 0);
  if (!cq_) throw std::runtime_error("verbs transport: ibv_create_cq failed");
  // one reliable-connected queue pair per peer, numbers published with the endpoint (caps as in the reference: rdma_utils.cc:499-505)
  qps_.assign(world_, nullptr);
  qp_state_.assign(world_, IBV_QPS_RESET);
  remote_.assign(world_, Remote{});
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    ibv_qp_init_attr ia;
    std::memset(&ia, 0, sizeof(ia));
    ia.send_cq = static_cast<ibv_cq*>(cq_);
    ia.recv_cq = static_cast<ibv_cq*>(cq_);
    ia.qp_type = IBV_QPT_RC;
    ia.cap.max_send_wr = 1024;
    ia.cap.max_recv_wr = 1024;
    ia.cap.max_send_sge = 1;
    ia.cap.max_recv_sge = 1;
    ia.sq_sig_all = 0;
    ibv_qp* qp = api_->create_qp(static_cast<ibv_pd*>(pd_), &ia);
    if (!qp) throw std::runtime_error("verbs transport: ibv_create_qp failed");
    qps_[r] = qp;
    ibv_qp_attr a;
    std::memset(&a, 0, sizeof(a));
    a.qp_state = IBV_QPS_INIT;
    a.pkey_index = 0;
    a.port_num = static_cast<uint8_t>(port_);
    a.qp_access_flags = kAccess;
    if (api_->modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS) != 0)
      throw std::runtime_error("verbs transport: queue pair did not reach INIT");
    qp_state_[r] = IBV_QPS_INIT;
  }
  bounce_mem_.assign(kBounceBytes + 64, 0);
  ibv_mr* mr = api_->reg_mr(static_cast<ibv_pd*>(pd_), bounce_mem_.data(), bounce_mem_.size(), kAccess);
  if (!mr) throw std::runtime_error("verbs transport: cannot register the staging buffer");
  bounce_ = Region{mr, bounce_mem_.data(), bounce_mem_.size(), mr->lkey, mr->rkey};
  active_ = true;
  PCCL_LOG_INFO("verbs transport: rank %d on port %d, lid %u, %d queue pairs", rank_, port_, static_cast<unsigned>(lid_), world_ - 1);
  return endpoint();
}

std::string VerbsTransport::endpoint() const {
  Json j = Json::object();
  j.set("gid", encodeHex(gid_, 16));
  j.set("lid", static_cast<int64_t>(lid_));
  Json q = Json::array();
  for (int r = 0; r < world_; ++r) q.push(Json(static_cast<int64_t>(qps_[r] ? static_cast<ibv_qp*>(qps_[r])->qp_num : 0)));
  j.set("qpn", q);
  Json b = Json::array();
  for (auto& reg : regions_) {
    Json e = Json::object();
    e.set("addr", static_cast<uint64_t>(reinterpret_cast<uintptr_t>(reg.ptr)));
    e.set("rkey", static_cast<uint64_t>(reg.rkey));
    e.set("bytes", static_cast<uint64_t>(reg.bytes));
    b.push(e);
  }
  j.set("buffers", b);
  return j.dump();
}

uint32_t VerbsTransport::regBuffer(void* ptr, size_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  if (!active_) throw std::runtime_error("verbs transport: activate first");
  ibv_mr* mr = api_->reg_mr(static_cast<ibv_pd*>(pd_), ptr, bytes, kAccess);
  if (!mr) throw std::runtime_error("verbs transport: ibv_reg_mr failed");
  regions_.push_back(Region{mr, static_cast<char*>(ptr), bytes, mr->lkey, mr->rkey});
  return static_cast<uint32_t>(regions_.size() - 1);
}

void VerbsTransport::unregBuffer(uint32_t key) {
  std::lock_guard<std::mutex> g(mu_);
  if (key >= regions_.size() || !regions_[key].mr) return;
  api_->dereg_mr(static_cast<ibv_mr*>(regions_[key].mr));
  regions_[key] = Region{};
}

void VerbsTransport::regRemoteHandle(int peer, const std::string& doc) {
  if (peer < 0 || peer >= world_ || peer == rank_) throw std::runtime_error("verbs transport: bad peer");
  Json j = Json::parse(doc);
  Remote r;
  bool ok = false;
  std::string raw = decodeHexToString(j["gid"].asString(), &ok);
  if (!ok || raw.size() != 16) throw std::runtime_error("verbs transport: malformed gid in the peer's endpoint");
  std::memcpy(r.gid, raw.data(), 16);
  r.lid = static_cast<uint16_t>(j["lid"].asInt());
  const Json& q = j["qpn"];
  if (static_cast<int>(q.size()) != world_) throw std::runtime_error("verbs transport: the peer's endpoint is for another world size");
  r.qpn = static_cast<uint32_t>(q.at(static_cast<size_t>(rank_)).asInt());
  const Json& b = j["buffers"];
  for (size_t i = 0; i < b.size(); ++i)
    r.bufs.emplace_back(static_cast<uint64_t>(b.at(i)["addr"].asInt()), static_cast<uint32_t>(b.at(i)["rkey"].asInt()));
  r.known = true;
  std::lock_guard<std::mutex> g(mu_);
  remote_[peer] = r;
}

void VerbsTransport::connect(int peer) {
  std::lock_guard<std::mutex> g(mu_);
  if (peer < 0 || peer >= world_ || peer == rank_ || !qps_[peer]) throw std::runtime_error("verbs transport: bad peer");
  if (!remote_[peer].known) throw std::runtime_error("verbs transport: no endpoint known for peer " + std::to_string(peer));
  if (qp_state_[peer] == IBV_QPS_RTS) return;
  ibv_qp* qp = static_cast<ibv_qp*>(qps_[peer]);
  const Remote& r = remote_[peer];
  // INIT -> RTR (reference parameters: rdma_utils.cc:756-795)
  ibv_qp_attr a;
  std::memset(&a, 0, sizeof(a));
  a.qp_state = IBV_QPS_RTR;
  a.path_mtu = IBV_MTU_2048;
  a.dest_qp_num = r.qpn;
  a.rq_psn = 0;
  a.max_dest_rd_atomic = 1;
  a.min_rnr_timer = 12;
  a.ah_attr.dlid = r.lid;
  a.ah_attr.sl = 0;
  a.ah_attr.src_path_bits = 0;
  a.ah_attr.port_num = static_cast<uint8_t>(port_);
  bool any = false;
  for (int i = 0; i < 16; ++i) any = any || r.gid[i] != 0;
  if (any) {                                    // RoCE and routed fabrics address by GID
    a.ah_attr.is_global = 1;
    std::memcpy(a.ah_attr.grh.dgid.raw, r.gid, 16);
    a.ah_attr.grh.sgid_index = static_cast<uint8_t>(gid_index_);
    a.ah_attr.grh.hop_limit = 64;
  }
  if (api_->modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC |
                                  IBV_QP_MIN_RNR_TIMER) != 0)
    throw std::runtime_error("verbs transport: queue pair did not reach RTR");
  qp_state_[peer] = IBV_QPS_RTR;
  // RTR -> RTS (rdma_utils.cc:797-820)
  std::memset(&a, 0, sizeof(a));
  a.qp_state = IBV_QPS_RTS;
  a.timeout = 14;
  a.retry_cnt = 7;
  a.rnr_retry = 7;
  a.sq_psn = 0;
  a.max_rd_atomic = 1;
  if (api_->modify_qp(qp, &a, IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC) != 0)
    throw std::runtime_error("verbs transport: queue pair did not reach RTS");
  qp_state_[peer] = IBV_QPS_RTS;
}

void VerbsTransport::disconnect(int peer) {
  std::lock_guard<std::mutex> g(mu_);
  if (peer < 0 || peer >= static_cast<int>(qps_.size()) || !qps_[peer]) return;
  ibv_qp_attr a;
  std::memset(&a, 0, sizeof(a));
  a.qp_state = IBV_QPS_RESET;
  api_->modify_qp(static_cast<ibv_qp*>(qps_[peer]), &a, IBV_QP_STATE);
  qp_state_[peer] = IBV_QPS_RESET;
}

std::string VerbsTransport::queuePairState(int peer) const {
  std::lock_guard<std::mutex> g(mu_);
  if (peer < 0 || peer >= static_cast<int>(qp_state_.size()) || !qps_[peer]) return "none";
  return stateName(qp_state_[peer]);
}

const VerbsTransport::Region* VerbsTransport::findLocal(const void* p, uint64_t bytes) const {
  const char* c = static_cast<const char*>(p);
  for (auto& r : regions_)
    if (r.mr && c >= r.ptr && c + bytes <= r.ptr + r.bytes) return &r;
  return nullptr;
}

// caller holds mu_: one work request in flight per transport keeps the completion matching trivial
bool VerbsTransport::postAndWait(int peer, void* wr_v) {
  ibv_send_wr* wr = static_cast<ibv_send_wr*>(wr_v);
  ibv_qp* qp = static_cast<ibv_qp*>(qps_[peer]);
  ibv_context* ctx = static_cast<ibv_context*>(ctx_);
  if (!ctx->ops.post_send || !ctx->ops.poll_cq) return false;
  ibv_send_wr* bad = nullptr;
  if (ctx->ops.post_send(qp, wr, &bad) != 0) return false;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms_);
  for (int spins = 0;; ++spins) {
    ibv_wc wc;
    std::memset(&wc, 0, sizeof(wc));
    int n = ctx->ops.poll_cq(static_cast<ibv_cq*>(cq_), 1, &wc);
    if (n < 0) return false;
    if (n == 1) {
      if (wc.status != IBV_WC_SUCCESS) {
        PCCL_LOG_ERROR("verbs transport: work request to rank %d completed with status %d", peer, wc.status);
        return false;
      }
      return true;
    }
    if ((spins & 1023) == 1023) {
      if (std::chrono::steady_clock::now() >= deadline) return false;
      std::this_thread::yield();
    }
  }
}

bool VerbsTransport::put(int peer, uint32_t key, uint64_t off, const void* src, uint64_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  if (!active_ || peer < 0 || peer >= world_ || !qps_[peer] || qp_state_[peer] != IBV_QPS_RTS) return false;
  const Remote& r = remote_[peer];
  if (key >= r.bufs.size()) return false;
  const char* s = static_cast<const char*>(src);
  uint64_t done = 0;
  while (done < bytes) {
    const Region* local = findLocal(s + done, bytes - done);
    uint64_t n = bytes - done;
    ibv_sge sge;
    if (local) {                          // registered memory goes out as it is, in pieces the 32-bit length can hold
      if (n > (1ull << 30)) n = 1ull << 30;
      sge = ibv_sge{static_cast<uint64_t>(reinterpret_cast<uintptr_t>(s + done)), static_cast<uint32_t>(n), local->lkey};
    } else {
      if (n > kBounceBytes) n = kBounceBytes;
      std::memcpy(bounce_.ptr, s + done, n);
      sge = ibv_sge{static_cast<uint64_t>(reinterpret_cast<uintptr_t>(bounce_.ptr)), static_cast<uint32_t>(n), bounce_.lkey};
    }
    ibv_send_wr wr;
    std::memset(&wr, 0, sizeof(wr));
    wr.wr_id = done;
    wr.sg_list = &sge;
    wr.num_sge = 1;
    wr.opcode = IBV_WR_RDMA_WRITE;
    wr.send_flags = IBV_SEND_SIGNALED;
    wr.wr.rdma.remote_addr = r.bufs[key].first + off + done;
    wr.wr.rdma.rkey = r.bufs[key].second;
    if (!postAndWait(peer, &wr)) return false;
    done += n;
  }
  bytes_sent_.fetch_add(bytes);
  return true;
}

bool VerbsTransport::signal(int peer, uint32_t slot, uint64_t add) {
  std::lock_guard<std::mutex> g(mu_);
  if (!active_ || peer < 0 || peer >= world_ || !qps_[peer] || qp_state_[peer] != IBV_QPS_RTS) return false;
  const Remote& r = remote_[peer];
  if (sig_key_ >= r.bufs.size() || slot >= sig_count_) return false;
  char* result = bounce_.ptr + kBounceBytes;          // the old value lands here; nobody reads it
  result += (8 - reinterpret_cast<uintptr_t>(result) % 8) % 8;
  ibv_sge sge{static_cast<uint64_t>(reinterpret_cast<uintptr_t>(result)), 8, bounce_.lkey};
  ibv_send_wr wr;
  std::memset(&wr, 0, sizeof(wr));
  wr.sg_list = &sge;
  wr.num_sge = 1;
  wr.opcode = IBV_WR_ATOMIC_FETCH_AND_ADD;
  wr.send_flags = IBV_SEND_SIGNALED;
  wr.wr.atomic.remote_addr = r.bufs[sig_key_].first + sig_off_ + 8ull * slot;
  wr.wr.atomic.compare_add = add;
  wr.wr.atomic.rkey = r.bufs[sig_key_].second;
  return postAndWait(peer, &wr);
}

void VerbsTransport::shutdown() {
  std::lock_guard<std::mutex> g(mu_);
  if (!api_ || !api_->ok()) return;
  for (auto& q : qps_)
    if (q) api_->destroy_qp(static_cast<ibv_qp*>(q));
  qps_.clear();
  for (auto& r : regions_)
    if (r.mr) api_->dereg_mr(static_cast<ibv_mr*>(r.mr));
  regions_.clear();
  if (bounce_.mr) api_->dereg_mr(static_cast<ibv_mr*>(bounce_.mr));
  bounce_ = Region{};
  if (cq_) api_->destroy_cq(static_cast<ibv_cq*>(cq_));
  if (pd_) api_->dealloc_pd(static_cast<ibv_pd*>(pd_));
  if (ctx_) api_->close_device(static_cast<ibv_context*>(ctx_));
  cq_ = pd_ = ctx_ = nullptr;
  active_ = false;
}

}  // namespace pccl
