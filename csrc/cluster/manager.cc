#include "manager.h"

#include <chrono>

#include "../common/clock.h"
#include "../common/json.h"
#include "../common/log.h"
#include "wire.h"

namespace pccl {

std::string NodeMeta::serialize() const {
  Json j = Json::object();
  j.set("rank", rank_);
  Json cfg = Json::object();
  for (auto& kv : endpoint_configs_) cfg.set(kv.first, kv.second);
  j.set("endpoint_configs", cfg);
  return j.dump();
}

bool NodeMeta::deserialize(const std::string& text, NodeMeta* out) {
  try {
    Json j = Json::parse(text);
    if (!j["rank"].isNumber() || !j["endpoint_configs"].isObject()) return false;
    out->rank_ = static_cast<int>(j["rank"].asInt());
    out->endpoint_configs_.clear();
    for (auto& kv : j["endpoint_configs"].members()) out->endpoint_configs_[kv.first] = kv.second.asString();
    return true;
  } catch (const std::exception&) {
    return false;
  }
}

ClusterManager::ClusterManager(int rank, int world, std::map<std::string, std::string> cfg)
    : rank_(rank), world_(world) {
  local_.rank_ = rank;
  local_.endpoint_configs_ = std::move(cfg);
  nodes_[rank] = local_;
  daemon_.setCallback([this](const ClusterMessage& m) { onEvent(m); });
}

ClusterManager::~ClusterManager() { killDaemonServer(); }

bool ClusterManager::initializeDaemonServer(const std::string& master_endpoint) {
  std::string host;
  int port = 0;
  if (!wire::splitHostPort(master_endpoint, &host, &port)) {
    PCCL_LOG_ERROR("cluster: bad master endpoint '%s'", master_endpoint.c_str());
    return false;
  }
  master_endpoint_ = master_endpoint;
  bool is_master = rank_ == 0;
  if (!daemon_.start(rank_, host, port, is_master)) return false;
  if (is_master) return true;   // joiners learn the master's own meta from onEvent(JoinNode)
  return daemon_.connectToMaster(host, port, local_.serialize());
}

void ClusterManager::killDaemonServer() {
  if (!daemon_.running()) return;
  if (!daemon_.isMaster()) daemon_.disconnectFromMaster();
  daemon_.stop();
}

void ClusterManager::addOrUpdateNode(const NodeMeta& meta) {
  {
    std::lock_guard<std::mutex> g(mu_);
    nodes_[meta.rank_] = meta;
  }
  cv_.notify_all();
}

void ClusterManager::removeNode(int rank) {
  {
    std::lock_guard<std::mutex> g(mu_);
    nodes_.erase(rank);
  }
  cv_.notify_all();
}

std::map<int, NodeMeta> ClusterManager::nodes() {
  std::lock_guard<std::mutex> g(mu_);
  return nodes_;
}

std::vector<int> ClusterManager::aliveRanks() {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<int> out;
  for (auto& kv : nodes_) out.push_back(kv.first);
  return out;
}

bool ClusterManager::waitForWorld(int world, int timeout_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  return cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms),
                      [&] { return static_cast<int>(nodes_.size()) >= world; });
}

bool ClusterManager::waitForDeparture(int rank, int timeout_ms) {
  std::unique_lock<std::mutex> lk(mu_);
  return cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return nodes_.count(rank) == 0; });
}

void ClusterManager::updateLocalMeta(const std::map<std::string, std::string>& cfg) {
  for (auto& kv : cfg) local_.endpoint_configs_[kv.first] = kv.second;
  addOrUpdateNode(local_);
  ClusterMessage m;
  m.event_type = ClusterEventType::UpdateNode;
  m.source_rank = rank_;
  m.target_rank = -1;
  m.data = local_.serialize();
  m.timestamp = nowNanos();
  if (daemon_.isMaster()) daemon_.broadcastMessage(m);
  else daemon_.sendMessage(m);
}

std::map<int, int> ClusterManager::resizeWorld() {
  std::map<int, int> mapping;
  {
    std::lock_guard<std::mutex> g(mu_);
    int next = 0;
    for (auto& kv : nodes_) mapping[kv.first] = next++;
    last_resize_ = mapping;
    world_ = next;
  }
  Json j = Json::object();
  j.set("world", static_cast<int>(mapping.size()));
  Json m = Json::object();
  for (auto& kv : mapping) m.set(std::to_string(kv.first), kv.second);
  j.set("mapping", m);
  ClusterMessage msg;
  msg.event_type = ClusterEventType::ResizeWorld;
  msg.source_rank = rank_;
  msg.target_rank = -1;
  msg.data = j.dump();
  msg.timestamp = nowNanos();
  daemon_.broadcastMessage(msg);
  cv_.notify_all();
  return mapping;
}

std::map<int, int> ClusterManager::lastResize() {
  std::lock_guard<std::mutex> g(mu_);
  return last_resize_;
}

void ClusterManager::onEvent(const ClusterMessage& msg) {
  switch (msg.event_type) {
    case ClusterEventType::JoinNode:
    case ClusterEventType::UpdateNode: {
      NodeMeta meta;
      if (NodeMeta::deserialize(msg.data, &meta)) {
        addOrUpdateNode(meta);
        if (daemon_.isMaster() && msg.event_type == ClusterEventType::JoinNode) {
          // a joiner must also learn the master's own meta
          ClusterMessage me;
          me.event_type = ClusterEventType::JoinNode;
          me.source_rank = rank_;
          me.target_rank = meta.rank_;
          me.data = local_.serialize();
          me.timestamp = nowNanos();
          daemon_.sendMessage(me);
        }
      } else {
        PCCL_LOG_WARN("cluster: unreadable node meta from rank %d", msg.source_rank);
      }
      break;
    }
    case ClusterEventType::QuitNode:
      removeNode(msg.source_rank);
      break;
    case ClusterEventType::ResizeWorld: {
      try {
        Json j = Json::parse(msg.data);
        std::lock_guard<std::mutex> g(mu_);
        last_resize_.clear();
        for (auto& kv : j["mapping"].members()) last_resize_[std::stoi(kv.first)] = static_cast<int>(kv.second.asInt());
        world_ = static_cast<int>(j["world"].asInt(world_));
      } catch (const std::exception&) {
      }
      cv_.notify_all();
      break;
    }
    case ClusterEventType::BeReplaced:
      PCCL_LOG_WARN("cluster: rank %d has been replaced by a new process", rank_);
      break;
    default:
      break;
  }
  if (on_change_) on_change_(msg.event_type, msg.source_rank);
}

}  // namespace pccl
