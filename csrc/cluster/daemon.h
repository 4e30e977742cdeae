// Cluster control plane: a TCP star (master accepts, workers connect) that carries membership
// events as framed JSON messages.
//
// Same role and vocabulary as the reference daemon (include/cluster/daemon.h:16-94,
// csrc/cluster/daemon.cc:1-299): ClusterMessage{event_type, data, source_rank, target_rank,
// timestamp}; events ResizeWorld, JoinSelf, QuitSelf, ReplaceOld, BeReplaced, JoinNode, QuitNode,
// UpdateNode; a callback runs on a worker thread.  The reference only ever produces
// JoinSelf/QuitSelf, drops read errors silently and has no liveness detection; here the master
// relays joins/updates/quits to everyone, every worker sends heartbeats, and a silent or closed
// peer is turned into a QuitNode event for the survivors (failure detection on the host; no GPU
// is involved).  Plain POSIX sockets and threads (the reference's asio is an empty submodule).
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace pccl {

enum class ClusterEventType : int {
  ResizeWorld = 0, JoinSelf, QuitSelf, ReplaceOld, BeReplaced, JoinNode, QuitNode, UpdateNode,
  Heartbeat   // internal: never delivered to the callback
};
const char* eventName(ClusterEventType t);

struct ClusterMessage {
  ClusterEventType event_type = ClusterEventType::Heartbeat;
  std::string data;          // event payload (usually a JSON document)
  int source_rank = -1;
  int target_rank = -1;      // -1 = everyone
  uint64_t timestamp = 0;    // ns since epoch at the sender
  std::string serialize() const;
  static bool deserialize(const std::string& text, ClusterMessage* out);
};

class Daemon {
 public:
  using EventCallback = std::function<void(const ClusterMessage&)>;
  Daemon();
  ~Daemon();

  void setCallback(EventCallback cb) { callback_ = std::move(cb); }
  // Master: binds host:port (port 0 = ephemeral) and accepts.  Worker: only starts the threads.
  bool start(int rank, const std::string& host, int port, bool is_master);
  void stop();
  bool running() const { return running_.load(); }
  bool isMaster() const { return is_master_; }
  int port() const { return port_; }

  // Worker side.
  bool connectToMaster(const std::string& host, int port, const std::string& join_payload, int timeout_ms = 30000);
  void disconnectFromMaster();   // graceful: sends QuitSelf first

  // Worker -> master, or master -> one worker (target_rank) / all workers (target_rank = -1).
  bool sendMessage(const ClusterMessage& msg);
  bool broadcastMessage(const ClusterMessage& msg, int except_rank = -1);

  // Test hooks (host-side fault injection): stop heartbeating / drop the socket without QuitSelf.
  void injectSilence(bool on) { silent_.store(on); }
  void injectAbruptClose();

  std::vector<int> connectedRanks();

 private:
  struct Peer {
    int fd = -1;
    int rank = -1;
    std::atomic<uint64_t> last_seen_ns{0};
    std::mutex send_mu;
    std::atomic<bool> open{true};
  };
  void acceptLoop();
  void readerLoop(std::shared_ptr<Peer> peer);
  void workerLoop();
  void heartbeatLoop();
  void enqueue(ClusterMessage msg);
  void masterHandle(std::shared_ptr<Peer> peer, ClusterMessage& msg);
  void declareGone(int rank, const char* why);
  bool sendTo(Peer& p, const ClusterMessage& msg);

  EventCallback callback_;
  int rank_ = -1;
  bool is_master_ = false;
  int listen_fd_ = -1;
  int port_ = 0;
  std::atomic<bool> running_{false};
  std::atomic<bool> silent_{false};
  std::thread accept_thread_, worker_thread_, heartbeat_thread_;
  std::mutex peers_mu_;
  std::map<int, std::shared_ptr<Peer>> peers_;          // master: by worker rank
  std::vector<std::shared_ptr<Peer>> anonymous_;        // master: accepted, not yet joined
  std::vector<std::shared_ptr<Peer>> graveyard_;        // replaced or departed peers, closed at stop()
  std::vector<std::thread> readers_;                    // joined at stop(); peers hold no thread
  void spawnReader(std::shared_ptr<Peer> peer);
  std::shared_ptr<Peer> master_;                        // worker: connection to the master
  std::map<int, std::string> join_payloads_;            // master: NodeMeta of every member
  std::mutex queue_mu_;
  std::condition_variable queue_cv_;
  std::deque<ClusterMessage> queue_;
  int heartbeat_ms_ = 200;
  int heartbeat_misses_ = 10;
};

}  // namespace pccl
