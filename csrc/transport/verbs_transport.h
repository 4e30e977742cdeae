// InfiniBand / RoCE data plane over reliable-connected queue pairs.
//
// Counterpart of the reference's verbs plugin (include/plugins/rdma_executor/utils/rdma_utils.h:15-319,
// csrc/plugins/rdma_executor/utils/rdma_utils.cc: a dlopen'd libibverbs, move-only wrappers for device list, context,
// protection domain, completion queue, memory region and queue pair, the INIT -> RTR -> RTS bring-up at :695-820, and a
// VerbsManager that nothing ever called).  Here the same life cycle sits behind the interface the engine already uses
// for its TCP fallback (activate -> endpoint document, regBuffer, regRemoteHandle, connect, put, signal):
//   * a PUT is an RDMA WRITE into the peer's registered heap; memory that is not registered goes through a registered
//     bounce buffer in 1 MiB pieces;
//   * a SIGNAL is an 8-byte RDMA fetch-and-add on the peer's signal word.  On one RC queue pair the atomic is ordered
//     behind the writes posted before it, which is the only ordering the instruction streams need;
//   * one queue pair per peer is created up front (its number travels in the endpoint document), `connect` moves it to
//     RTR and RTS with the reference's parameters (MTU 2048, 7 retries, timeout 14, RNR timer 12).
// Every completion is polled with a deadline.  The library is loaded at run time (PCCL_IBVERBS_LIB overrides its name:
// the CPU tests point it at a stand-in that moves the bytes inside the process); the ABI it is called through is
// declared in verbs_abi.h.  Off unless PCCL_TRANSPORT=verbs.
#pragma once
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../base/device.h"

namespace pccl {

struct VerbsApi;      // the resolved library entry points

class VerbsTransport : public RemoteCommunicatorBase {
 public:
  VerbsTransport(int rank, int world);
  ~VerbsTransport() override;
  // True when the library loads and shows at least one device; *why says what is missing otherwise.
  static bool probe(std::string* why);

  bool remoteCommAvailable() override;
  std::string activate() override;                        // endpoint document: gid, lid, one queue-pair number per rank, buffers
  uint32_t regBuffer(void* ptr, size_t bytes) override;   // registers a memory region; key = registration order
  void unregBuffer(uint32_t key) override;
  void regRemoteHandle(int peer, const std::string& endpoint) override;
  void connect(int peer) override;                        // RESET/INIT -> RTR -> RTS of the queue pair kept for `peer`
  void disconnect(int peer) override;
  bool put(int peer, uint32_t remote_key, uint64_t remote_off, const void* src, uint64_t bytes) override;
  bool signal(int peer, uint32_t slot, uint64_t add) override;
  uint64_t bytesSent() const override { return bytes_sent_.load(); }

  // Signal word `slot` of a peer is the 8 bytes at `offset + 8 * slot` of that peer's buffer `key`.
  void setSignalRegion(uint32_t key, uint64_t offset, uint32_t count) { sig_key_ = key; sig_off_ = offset; sig_count_ = count; }
  // The endpoint document again, now with the buffers registered since activate().
  std::string endpoint() const;
  std::string queuePairState(int peer) const;             // "RESET", "INIT", "RTR", "RTS" (for tests and diagnostics)
  void shutdown();

 private:
  struct Region { void* mr = nullptr; char* ptr = nullptr; size_t bytes = 0; uint32_t lkey = 0, rkey = 0; };
  struct Remote { bool known = false; uint8_t gid[16] = {0}; uint16_t lid = 0; uint32_t qpn = 0; std::vector<std::pair<uint64_t, uint32_t>> bufs; };
  bool postAndWait(int peer, void* wr);                   // one signaled work request, polled to completion
  const Region* findLocal(const void* p, uint64_t bytes) const;

  int rank_, world_;
  std::shared_ptr<VerbsApi> api_;
  void* ctx_ = nullptr;      // ibv_context*
  void* pd_ = nullptr;       // ibv_pd*
  void* cq_ = nullptr;       // ibv_cq*
  std::vector<void*> qps_;   // ibv_qp* per peer rank (null for our own)
  std::vector<int> qp_state_;
  std::vector<Remote> remote_;
  std::vector<Region> regions_;
  Region bounce_;            // 1 MiB staging + 8 bytes for atomic results
  std::vector<char> bounce_mem_;
  int port_ = 1, gid_index_ = 0;
  uint16_t lid_ = 0;
  uint8_t gid_[16] = {0};
  uint32_t sig_key_ = 0, sig_count_ = 0;
  uint64_t sig_off_ = 0;
  int timeout_ms_ = 30000;
  mutable std::mutex mu_;
  std::atomic<uint64_t> bytes_sent_{0};
  bool active_ = false;
};

}  // namespace pccl
