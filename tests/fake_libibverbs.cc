// Stand-in for libibverbs, for tests on machines without an InfiniBand adapter.  It implements the entry points that
// csrc/transport/verbs_transport.cc resolves, against the ABI of csrc/transport/verbs_abi.h, and moves the bytes inside
// the process: an RDMA WRITE is a memcpy into the target address after the rkey and range have been checked against the
// registered regions, a fetch-and-add is an atomic add.  It is strict about the queue-pair state machine (RESET -> INIT
// -> RTR -> RTS, each step with the attribute mask the real library demands) and keeps a log the tests read.
#include <atomic>
#include <cerrno>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../csrc/transport/verbs_abi.h"

struct ibv_device { char name[64]; };

namespace {
std::mutex g_mu;
struct FakeMr { ibv_mr mr; };
struct FakeCq { ibv_cq cq; std::deque<ibv_wc> done; };
struct FakeQp { ibv_qp qp; FakeCq* scq; uint32_t dest_qpn = 0; int access = 0; };
std::map<uint32_t, FakeQp*> g_qps;
std::vector<FakeMr*> g_mrs;
std::string g_log;
uint32_t g_next_qpn = 100, g_next_key = 1000;
int g_devices = 1;
ibv_device g_dev = {"fake0"};
ibv_device* g_list[2] = {&g_dev, nullptr};

void logf(const std::string& s) { g_log += s + ";"; }

FakeMr* findMr(uint32_t rkey, uint64_t addr, uint64_t len) {
  for (FakeMr* m : g_mrs)
    if (m && m->mr.rkey == rkey && addr >= reinterpret_cast<uintptr_t>(m->mr.addr) &&
        addr + len <= reinterpret_cast<uintptr_t>(m->mr.addr) + m->mr.length)
      return m;
  return nullptr;
}
bool localOk(uint32_t lkey, uint64_t addr, uint64_t len) {
  for (FakeMr* m : g_mrs)
    if (m && m->mr.lkey == lkey && addr >= reinterpret_cast<uintptr_t>(m->mr.addr) &&
        addr + len <= reinterpret_cast<uintptr_t>(m->mr.addr) + m->mr.length)
      return true;
  return false;
}

int fake_poll_cq(ibv_cq* cq, int n, ibv_wc* wc) {
  std::lock_guard<std::mutex> g(g_mu);
  FakeCq* f = reinterpret_cast<FakeCq*>(cq);
  int k = 0;
  while (k < n && !f->done.empty()) {
    wc[k++] = f->done.front();
    f->done.pop_front();
  }
  return k;
}

int fake_post_send(ibv_qp* qp, ibv_send_wr* wr, ibv_send_wr** bad) {
  std::lock_guard<std::mutex> g(g_mu);
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  for (; wr; wr = wr->next) {
    ibv_wc wc;
    std::memset(&wc, 0, sizeof(wc));
    wc.wr_id = wr->wr_id;
    wc.qp_num = q->qp.qp_num;
    auto fail = [&](int status, const char* why) {
      wc.status = status;
      logf(std::string("error:") + why);
    };
    if (q->qp.state != IBV_QPS_RTS) {
      if (bad) *bad = wr;
      logf("post_send-before-RTS");
      return EINVAL;
    }
    auto it = g_qps.find(q->dest_qpn);
    FakeQp* peer = it == g_qps.end() ? nullptr : it->second;
    if (!peer || peer->qp.state < IBV_QPS_RTR || peer->dest_qpn != q->qp.qp_num) fail(12, "peer-not-ready");       // retry exceeded
    else if (wr->num_sge != 1 || !localOk(wr->sg_list[0].lkey, wr->sg_list[0].addr, wr->sg_list[0].length)) fail(4, "local-protection");
    else if (wr->opcode == IBV_WR_RDMA_WRITE) {
      if (!(peer->access & IBV_ACCESS_REMOTE_WRITE) || !findMr(wr->wr.rdma.rkey, wr->wr.rdma.remote_addr, wr->sg_list[0].length)) fail(10, "remote-access");
      else {
        std::memcpy(reinterpret_cast<void*>(wr->wr.rdma.remote_addr), reinterpret_cast<void*>(wr->sg_list[0].addr), wr->sg_list[0].length);
        wc.byte_len = wr->sg_list[0].length;
        logf("write:" + std::to_string(wr->sg_list[0].length));
      }
    } else if (wr->opcode == IBV_WR_ATOMIC_FETCH_AND_ADD) {
      if (!(peer->access & IBV_ACCESS_REMOTE_ATOMIC) || wr->sg_list[0].length != 8 || (wr->wr.atomic.remote_addr & 7) ||
          !findMr(wr->wr.atomic.rkey, wr->wr.atomic.remote_addr, 8)) fail(10, "remote-access");
      else {
        auto* word = reinterpret_cast<std::atomic<uint64_t>*>(wr->wr.atomic.remote_addr);
        uint64_t old = word->fetch_add(wr->wr.atomic.compare_add, std::memory_order_acq_rel);
        std::memcpy(reinterpret_cast<void*>(wr->sg_list[0].addr), &old, 8);
        logf("faa");
      }
    } else fail(9, "unsupported-opcode");
    if ((wr->send_flags & IBV_SEND_SIGNALED) || wc.status != 0) q->scq->done.push_back(wc);
  }
  return 0;
}
int fake_post_recv(ibv_qp*, ibv_recv_wr*, ibv_recv_wr**) { return 0; }
int fake_req_notify(ibv_cq*, int) { return 0; }
}  // namespace

extern "C" {
__attribute__((visibility("default"))) ibv_device** ibv_get_device_list(int* n) { if (n) *n = g_devices; return g_devices ? g_list : nullptr; }
__attribute__((visibility("default"))) void ibv_free_device_list(ibv_device**) {}
__attribute__((visibility("default"))) const char* ibv_get_device_name(ibv_device* d) { return d->name; }
__attribute__((visibility("default"))) ibv_context* ibv_open_device(ibv_device* d) {
  ibv_context* c = new ibv_context();
  std::memset(c, 0, sizeof(*c));
  c->device = d;
  c->ops.poll_cq = fake_poll_cq;
  c->ops.post_send = fake_post_send;
  c->ops.post_recv = fake_post_recv;
  c->ops.req_notify_cq = fake_req_notify;
  std::lock_guard<std::mutex> g(g_mu);
  logf("open");
  return c;
}
__attribute__((visibility("default"))) int ibv_close_device(ibv_context* c) { delete c; return 0; }
__attribute__((visibility("default"))) int ibv_query_port(ibv_context*, uint8_t port, ibv_port_attr* a) {
  if (port != 1) return EINVAL;
  a->state = 4;
  a->active_mtu = IBV_MTU_4096;
  a->lid = 7;
  return 0;
}
__attribute__((visibility("default"))) int ibv_query_gid(ibv_context*, uint8_t, int index, ibv_gid* g) {
  std::memset(g, 0, sizeof(*g));
  g->raw[0] = 0xfe; g->raw[1] = 0x80; g->raw[15] = static_cast<uint8_t>(1 + index);
  return 0;
}
__attribute__((visibility("default"))) ibv_pd* ibv_alloc_pd(ibv_context* c) { ibv_pd* p = new ibv_pd(); p->context = c; p->handle = 1; return p; }
__attribute__((visibility("default"))) int ibv_dealloc_pd(ibv_pd* p) { delete p; return 0; }
__attribute__((visibility("default"))) ibv_mr* ibv_reg_mr(ibv_pd* pd, void* addr, size_t len, int access) {
  (void)access;
  FakeMr* m = new FakeMr();
  std::memset(&m->mr, 0, sizeof(m->mr));
  m->mr.context = pd->context; m->mr.pd = pd; m->mr.addr = addr; m->mr.length = len;
  std::lock_guard<std::mutex> g(g_mu);
  m->mr.lkey = g_next_key++; m->mr.rkey = g_next_key++;
  g_mrs.push_back(m);
  return &m->mr;
}
__attribute__((visibility("default"))) int ibv_dereg_mr(ibv_mr* mr) {
  std::lock_guard<std::mutex> g(g_mu);
  for (auto& m : g_mrs)
    if (m && &m->mr == mr) { delete m; m = nullptr; return 0; }
  return EINVAL;
}
__attribute__((visibility("default"))) ibv_cq* ibv_create_cq(ibv_context* c, int cqe, void*, ibv_comp_channel*, int) {
  FakeCq* f = new FakeCq();
  std::memset(&f->cq, 0, sizeof(f->cq));
  f->cq.context = c; f->cq.cqe = cqe;
  return &f->cq;
}
__attribute__((visibility("default"))) int ibv_destroy_cq(ibv_cq* cq) { delete reinterpret_cast<FakeCq*>(cq); return 0; }
__attribute__((visibility("default"))) ibv_qp* ibv_create_qp(ibv_pd* pd, ibv_qp_init_attr* ia) {
  if (ia->qp_type != IBV_QPT_RC || !ia->send_cq) return nullptr;
  FakeQp* q = new FakeQp();
  std::memset(&q->qp, 0, sizeof(q->qp));
  q->qp.context = pd->context; q->qp.pd = pd; q->qp.send_cq = ia->send_cq; q->qp.recv_cq = ia->recv_cq;
  q->qp.qp_type = IBV_QPT_RC; q->qp.state = IBV_QPS_RESET;
  q->scq = reinterpret_cast<FakeCq*>(ia->send_cq);
  std::lock_guard<std::mutex> g(g_mu);
  q->qp.qp_num = g_next_qpn++;
  g_qps[q->qp.qp_num] = q;
  return &q->qp;
}
__attribute__((visibility("default"))) int ibv_destroy_qp(ibv_qp* qp) {
  std::lock_guard<std::mutex> g(g_mu);
  g_qps.erase(qp->qp_num);
  delete reinterpret_cast<FakeQp*>(qp);
  return 0;
}
__attribute__((visibility("default"))) int ibv_modify_qp(ibv_qp* qp, ibv_qp_attr* a, int mask) {
  std::lock_guard<std::mutex> g(g_mu);
  FakeQp* q = reinterpret_cast<FakeQp*>(qp);
  if (!(mask & IBV_QP_STATE)) return EINVAL;
  const int init_mask = IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS;
  const int rtr_mask = IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN | IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER;
  const int rts_mask = IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN | IBV_QP_MAX_QP_RD_ATOMIC;
  const std::string id = "qp" + std::to_string(q->qp.qp_num);
  switch (a->qp_state) {
    case IBV_QPS_RESET: q->qp.state = IBV_QPS_RESET; q->dest_qpn = 0; logf(id + ":RESET"); return 0;
    case IBV_QPS_INIT:
      if (q->qp.state != IBV_QPS_RESET || mask != init_mask || a->port_num != 1) { logf(id + ":bad-INIT"); return EINVAL; }
      q->access = static_cast<int>(a->qp_access_flags);
      q->qp.state = IBV_QPS_INIT; logf(id + ":INIT"); return 0;
    case IBV_QPS_RTR:
      if (q->qp.state != IBV_QPS_INIT || mask != rtr_mask || a->path_mtu < IBV_MTU_256 || a->path_mtu > IBV_MTU_4096 || a->ah_attr.port_num != 1 ||
          (a->ah_attr.is_global && a->ah_attr.grh.hop_limit == 0)) { logf(id + ":bad-RTR"); return EINVAL; }
      q->dest_qpn = a->dest_qp_num;
      q->qp.state = IBV_QPS_RTR; logf(id + ":RTR"); return 0;
    case IBV_QPS_RTS:
      if (q->qp.state != IBV_QPS_RTR || mask != rts_mask || a->retry_cnt > 7 || a->rnr_retry > 7) { logf(id + ":bad-RTS"); return EINVAL; }
      q->qp.state = IBV_QPS_RTS; logf(id + ":RTS"); return 0;
    default: return EINVAL;
  }
}

// ---- what the tests look at ----
__attribute__((visibility("default"))) const char* fake_ibv_log() { static std::string copy; std::lock_guard<std::mutex> g(g_mu); copy = g_log; return copy.c_str(); }
__attribute__((visibility("default"))) void fake_ibv_set_devices(int n) { g_devices = n; }
}
