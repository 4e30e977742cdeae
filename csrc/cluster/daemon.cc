#include "daemon.h"

#include <chrono>

#include "../common/clock.h"
#include "../common/env.h"
#include "../common/json.h"
#include "../common/log.h"
#include "wire.h"

namespace pccl {

static const char* kEventNames[] = {"ResizeWorld", "JoinSelf", "QuitSelf", "ReplaceOld", "BeReplaced",
                                    "JoinNode", "QuitNode", "UpdateNode", "Heartbeat"};
constexpr uint32_t kFrameCluster = 1;

const char* eventName(ClusterEventType t) { return kEventNames[static_cast<int>(t)]; }

std::string ClusterMessage::serialize() const {
  Json j = Json::object();
  j.set("event_type", static_cast<int>(event_type));
  j.set("data", data);
  j.set("source_rank", source_rank);
  j.set("target_rank", target_rank);
  j.set("timestamp", timestamp);
  return j.dump();
}

bool ClusterMessage::deserialize(const std::string& text, ClusterMessage* out) {
  try {
    Json j = Json::parse(text);
    int64_t e = j["event_type"].asInt(-1);
    if (e < 0 || e > static_cast<int>(ClusterEventType::Heartbeat)) return false;
    out->event_type = static_cast<ClusterEventType>(e);
    out->data = j["data"].asString();
    out->source_rank = static_cast<int>(j["source_rank"].asInt(-1));
    out->target_rank = static_cast<int>(j["target_rank"].asInt(-1));
    out->timestamp = static_cast<uint64_t>(j["timestamp"].asInt(0));
    return true;
  } catch (const std::exception&) {
    return false;
  }
}

Daemon::Daemon() {
  heartbeat_ms_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_HEARTBEAT_MS", 200));
  heartbeat_misses_ = static_cast<int>(LaunchEnvironments::getInt("PCCL_HEARTBEAT_MISSES", 10));
}

Daemon::~Daemon() { stop(); }

bool Daemon::start(int rank, const std::string& host, int port, bool is_master) {
  if (running_.load()) return true;
  rank_ = rank;
  is_master_ = is_master;
  if (is_master) {
    port_ = port;
    listen_fd_ = wire::tcpListen(host, &port_);
    if (listen_fd_ < 0) {
      PCCL_LOG_ERROR("daemon: cannot listen on %s:%d", host.c_str(), port);
      return false;
    }
  }
  running_.store(true);
  worker_thread_ = std::thread([this] { workerLoop(); });
  heartbeat_thread_ = std::thread([this] { heartbeatLoop(); });
  if (is_master) accept_thread_ = std::thread([this] { acceptLoop(); });
  return true;
}

void Daemon::spawnReader(std::shared_ptr<Peer> peer) {
  std::lock_guard<std::mutex> g(peers_mu_);
  readers_.emplace_back([this, peer] { readerLoop(peer); });
}

void Daemon::stop() {
  if (!running_.exchange(false)) return;
  queue_cv_.notify_all();
  if (listen_fd_ >= 0) wire::shutdownFd(listen_fd_);
  if (accept_thread_.joinable()) accept_thread_.join();   // after this no new reader can appear
  std::vector<std::shared_ptr<Peer>> all;
  std::vector<std::thread> readers;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    for (auto& kv : peers_) all.push_back(kv.second);
    for (auto& p : anonymous_) all.push_back(p);
    for (auto& p : graveyard_) all.push_back(p);
    if (master_) all.push_back(master_);
    readers.swap(readers_);
  }
  for (auto& p : all) {
    p->open.store(false);
    wire::shutdownFd(p->fd);
  }
  for (auto& t : readers)
    if (t.joinable()) t.join();
  if (heartbeat_thread_.joinable()) heartbeat_thread_.join();
  if (worker_thread_.joinable()) worker_thread_.join();
  {
    // a reader that was inside declareGone() may have moved its peer between the lists meanwhile
    std::lock_guard<std::mutex> g(peers_mu_);
    for (auto& kv : peers_) all.push_back(kv.second);
    for (auto& p : anonymous_) all.push_back(p);
    for (auto& p : graveyard_) all.push_back(p);
    peers_.clear();
    anonymous_.clear();
    graveyard_.clear();
    master_.reset();
  }
  for (auto& p : all) {
    if (p->fd >= 0) wire::closeFd(p->fd);
    p->fd = -1;
  }
  wire::closeFd(listen_fd_);
  listen_fd_ = -1;
}

bool Daemon::sendTo(Peer& p, const ClusterMessage& msg) {
  if (!p.open.load()) return false;
  std::string s = msg.serialize();
  std::lock_guard<std::mutex> g(p.send_mu);
  return wire::sendFrame(p.fd, kFrameCluster, s.data(), s.size());
}

bool Daemon::connectToMaster(const std::string& host, int port, const std::string& join_payload, int timeout_ms) {
  int fd = wire::tcpConnect(host, port, timeout_ms);
  if (fd < 0) {
    PCCL_LOG_ERROR("daemon: rank %d cannot reach master %s:%d", rank_, host.c_str(), port);
    return false;
  }
  auto peer = std::make_shared<Peer>();
  peer->fd = fd;
  peer->rank = 0;
  peer->last_seen_ns.store(monotonicNanos());
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    master_ = peer;
  }
  ClusterMessage join;
  join.event_type = ClusterEventType::JoinSelf;
  join.data = join_payload;
  join.source_rank = rank_;
  join.target_rank = 0;
  join.timestamp = nowNanos();
  if (!sendTo(*peer, join)) return false;
  spawnReader(peer);
  return true;
}

void Daemon::disconnectFromMaster() {
  std::shared_ptr<Peer> m;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    m = master_;
  }
  if (!m) return;
  ClusterMessage q;
  q.event_type = ClusterEventType::QuitSelf;
  q.source_rank = rank_;
  q.target_rank = 0;
  q.timestamp = nowNanos();
  sendTo(*m, q);
  m->open.store(false);
  wire::shutdownFd(m->fd);
}

void Daemon::injectAbruptClose() {
  std::shared_ptr<Peer> m;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    m = master_;
  }
  if (m) {
    m->open.store(false);
    wire::shutdownFd(m->fd);
  }
}

bool Daemon::sendMessage(const ClusterMessage& msg) {
  std::shared_ptr<Peer> p;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    if (is_master_) {
      auto it = peers_.find(msg.target_rank);
      if (it != peers_.end()) p = it->second;
    } else {
      p = master_;
    }
  }
  return p && sendTo(*p, msg);
}

bool Daemon::broadcastMessage(const ClusterMessage& msg, int except_rank) {
  if (!is_master_) return false;
  std::vector<std::shared_ptr<Peer>> all;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    for (auto& kv : peers_)
      if (kv.first != except_rank) all.push_back(kv.second);
  }
  bool ok = true;
  for (auto& p : all) ok = sendTo(*p, msg) && ok;
  return ok;
}

std::vector<int> Daemon::connectedRanks() {
  std::lock_guard<std::mutex> g(peers_mu_);
  std::vector<int> out;
  for (auto& kv : peers_) out.push_back(kv.first);
  return out;
}

void Daemon::acceptLoop() {
  while (running_.load()) {
    int fd = wire::acceptOne(listen_fd_, 100);
    if (fd < 0) continue;
    auto peer = std::make_shared<Peer>();
    peer->fd = fd;
    peer->last_seen_ns.store(monotonicNanos());
    {
      std::lock_guard<std::mutex> g(peers_mu_);
      anonymous_.push_back(peer);
    }
    spawnReader(peer);
  }
}

void Daemon::enqueue(ClusterMessage msg) {
  {
    std::lock_guard<std::mutex> g(queue_mu_);
    queue_.push_back(std::move(msg));
  }
  queue_cv_.notify_one();
}

void Daemon::declareGone(int rank, const char* why) {
  std::shared_ptr<Peer> p;
  {
    std::lock_guard<std::mutex> g(peers_mu_);
    auto it = peers_.find(rank);
    if (it == peers_.end()) return;
    p = it->second;
    peers_.erase(it);
    join_payloads_.erase(rank);
  }
  p->open.store(false);
  wire::shutdownFd(p->fd);
  PCCL_LOG_WARN("daemon: rank %d is gone (%s)", rank, why);
  ClusterMessage q;
  q.event_type = ClusterEventType::QuitNode;
  q.source_rank = rank;
  q.target_rank = -1;
  q.timestamp = nowNanos();
  q.data = why;
  broadcastMessage(q);
  enqueue(q);
  // its socket is closed in stop(); keep the object until then
  std::lock_guard<std::mutex> g(peers_mu_);
  graveyard_.push_back(p);
}

void Daemon::masterHandle(std::shared_ptr<Peer> peer, ClusterMessage& msg) {
  switch (msg.event_type) {
    case ClusterEventType::JoinSelf:
    case ClusterEventType::ReplaceOld: {
      std::shared_ptr<Peer> old;
      std::vector<std::pair<int, std::string>> known;
      {
        std::lock_guard<std::mutex> g(peers_mu_);
        auto it = peers_.find(msg.source_rank);
        if (it != peers_.end() && it->second != peer) old = it->second;
        peer->rank = msg.source_rank;
        peers_[msg.source_rank] = peer;
        for (auto a = anonymous_.begin(); a != anonymous_.end(); ++a)
          if (*a == peer) { anonymous_.erase(a); break; }
        for (auto& kv : join_payloads_)
          if (kv.first != msg.source_rank) known.emplace_back(kv.first, kv.second);
        join_payloads_[msg.source_rank] = msg.data;
        if (old) graveyard_.push_back(old);
      }
      if (old) {
        ClusterMessage br;
        br.event_type = ClusterEventType::BeReplaced;
        br.source_rank = 0;
        br.target_rank = msg.source_rank;
        br.timestamp = nowNanos();
        sendTo(*old, br);
        old->open.store(false);
        wire::shutdownFd(old->fd);
      }
      // tell the newcomer about everyone already here (the master included) ...
      for (auto& kv : known) {
        ClusterMessage jn;
        jn.event_type = ClusterEventType::JoinNode;
        jn.source_rank = kv.first;
        jn.target_rank = msg.source_rank;
        jn.data = kv.second;
        jn.timestamp = nowNanos();
        sendTo(*peer, jn);
      }
      // ... and everyone else about the newcomer
      ClusterMessage ann;
      ann.event_type = old ? ClusterEventType::UpdateNode : ClusterEventType::JoinNode;
      ann.source_rank = msg.source_rank;
      ann.target_rank = -1;
      ann.data = msg.data;
      ann.timestamp = nowNanos();
      broadcastMessage(ann, msg.source_rank);
      enqueue(ann);
      break;
    }
    case ClusterEventType::UpdateNode: {
      {
        std::lock_guard<std::mutex> g(peers_mu_);
        join_payloads_[msg.source_rank] = msg.data;
      }
      broadcastMessage(msg, msg.source_rank);
      enqueue(msg);
      break;
    }
    case ClusterEventType::QuitSelf:
      declareGone(msg.source_rank, "left");
      break;
    case ClusterEventType::Heartbeat:
      break;
    default:
      // ResizeWorld etc. from a worker: relay
      if (msg.target_rank < 0) broadcastMessage(msg, msg.source_rank);
      else if (msg.target_rank != rank_) { sendMessage(msg); break; }
      enqueue(msg);
  }
}

void Daemon::readerLoop(std::shared_ptr<Peer> peer) {
  while (running_.load() && peer->open.load()) {
    uint32_t kind = 0;
    std::string payload;
    if (!wire::recvFrame(peer->fd, &kind, &payload)) break;
    peer->last_seen_ns.store(monotonicNanos());
    ClusterMessage msg;
    if (kind != kFrameCluster || !ClusterMessage::deserialize(payload, &msg)) {
      PCCL_LOG_WARN("daemon: dropping malformed control message (%zu bytes)", payload.size());
      continue;
    }
    if (is_master_) {
      masterHandle(peer, msg);
    } else if (msg.event_type != ClusterEventType::Heartbeat) {
      enqueue(msg);
    }
  }
  bool was_open = peer->open.exchange(false);
  if (!running_.load()) return;
  if (is_master_) {
    if (peer->rank >= 0 && was_open) declareGone(peer->rank, "connection closed");
  } else if (was_open) {
    // the master vanished: report it locally as QuitNode(0)
    ClusterMessage q;
    q.event_type = ClusterEventType::QuitNode;
    q.source_rank = 0;
    q.data = "master connection closed";
    q.timestamp = nowNanos();
    enqueue(q);
  }
}

void Daemon::heartbeatLoop() {
  while (running_.load()) {
    std::this_thread::sleep_for(std::chrono::milliseconds(heartbeat_ms_));
    if (!running_.load()) break;
    if (!is_master_) {
      if (silent_.load()) continue;
      ClusterMessage hb;
      hb.event_type = ClusterEventType::Heartbeat;
      hb.source_rank = rank_;
      hb.target_rank = 0;
      hb.timestamp = nowNanos();
      sendMessage(hb);
    } else {
      uint64_t now = monotonicNanos();
      uint64_t limit = static_cast<uint64_t>(heartbeat_ms_) * heartbeat_misses_ * 1000000ull;
      std::vector<int> dead;
      {
        std::lock_guard<std::mutex> g(peers_mu_);
        for (auto& kv : peers_)
          if (now - kv.second->last_seen_ns.load() > limit) dead.push_back(kv.first);
      }
      for (int r : dead) declareGone(r, "heartbeat timeout");
    }
  }
}

void Daemon::workerLoop() {
  for (;;) {
    ClusterMessage msg;
    {
      std::unique_lock<std::mutex> lk(queue_mu_);
      queue_cv_.wait(lk, [this] { return !queue_.empty() || !running_.load(); });
      if (queue_.empty()) return;
      msg = std::move(queue_.front());
      queue_.pop_front();
    }
    if (callback_) {
      try {
        callback_(msg);
      } catch (const std::exception& e) {
        PCCL_LOG_ERROR("daemon: event callback threw: %s", e.what());
      }
    }
  }
}

}  // namespace pccl
