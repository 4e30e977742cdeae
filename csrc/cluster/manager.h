// Cluster membership: NodeMeta (a rank's endpoint document) and ClusterManager, which owns the
// daemon and the table of known nodes.  Counterpart of include/cluster/manager.h:9-28 (whose
// serialize() refers to a member that does not exist, csrc/cluster/manager.cc:10, and whose other
// methods are never defined).
#pragma once
#include <condition_variable>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "daemon.h"

namespace pccl {

struct NodeMeta {
  int rank_ = -1;
  std::map<std::string, std::string> endpoint_configs_;   // flat dotted keys, like the reference
  std::string serialize() const;
  static bool deserialize(const std::string& text, NodeMeta* out);
};

class ClusterManager {
 public:
  using MembershipCallback = std::function<void(ClusterEventType, int rank)>;
  ClusterManager(int rank, int world, std::map<std::string, std::string> local_config);
  ~ClusterManager();

  // Rank 0 listens on master_endpoint ("host:port"); other ranks connect to it and announce
  // themselves.  Returns once the daemon is up (not once everyone joined: see waitForWorld).
  bool initializeDaemonServer(const std::string& master_endpoint);
  void killDaemonServer();
  bool waitForWorld(int world, int timeout_ms);
  bool waitForDeparture(int rank, int timeout_ms);

  const NodeMeta& getLocalMeta() const { return local_; }
  void updateLocalMeta(const std::map<std::string, std::string>& cfg);   // re-announces (UpdateNode)
  void addOrUpdateNode(const NodeMeta& meta);
  void removeNode(int rank);
  std::map<int, NodeMeta> nodes();
  std::vector<int> aliveRanks();
  int world() const { return world_; }
  void setMembershipCallback(MembershipCallback cb) { on_change_ = std::move(cb); }
  // Master only: announce a new world made of the currently alive ranks (old rank -> new rank).
  std::map<int, int> resizeWorld();
  std::map<int, int> lastResize();
  Daemon& daemon() { return daemon_; }
  std::string masterEndpoint() const { return master_endpoint_; }

 private:
  void onEvent(const ClusterMessage& msg);
  int rank_, world_;
  NodeMeta local_;
  Daemon daemon_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::map<int, NodeMeta> nodes_;
  std::map<int, int> last_resize_;
  MembershipCallback on_change_;
  std::string master_endpoint_;
};

}  // namespace pccl
