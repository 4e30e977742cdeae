// Host/TCP data-plane transport.
//
// Plays the part the reference gives to its verbs plugin (csrc/plugins/rdma_executor/device.cc:
// 38-77, rdma_utils.*: activate -> publish an endpoint handle, register buffers, connect to a
// peer, post writes): here a "write" is a framed TCP message that the peer's receiver thread
// copies into the registered buffer, and a "notify" is a framed increment of one of the peer's
// signal words.  One connection per (sender, receiver) pair keeps PUT-then-SIGNAL ordered, which is
// the only ordering the instruction streams rely on.  This is the fallback used between hosts
// without InfiniBand and by CPU ranks when PCCL_TRANSPORT=tcp.
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "../base/device.h"

namespace pccl {

class TcpTransport : public RemoteCommunicatorBase {
 public:
  TcpTransport() = default;
  ~TcpTransport() override;
  bool remoteCommAvailable() override { return true; }
  std::string activate() override;                        // "host:port" of our receiver
  uint32_t regBuffer(void* ptr, size_t bytes) override;   // key = registration order (0,1,2..)
  void unregBuffer(uint32_t key) override;
  void regRemoteHandle(int peer, const std::string& endpoint) override;
  void connect(int peer) override;
  void disconnect(int peer) override;

  void setSignals(std::atomic<uint64_t>* signals, uint32_t count) { signals_ = signals; num_signals_ = count; }
  // Called by the receiver thread after the bytes of a PUT have landed in the registered buffer and before the next
  // frame of that connection is read -- so before the SIGNAL that follows the PUT takes effect.  A CUDA engine uses it
  // to move the bytes from its host shadow of the workspace on to the device.
  void setPutHook(std::function<void(uint32_t key, uint64_t off, uint64_t bytes)> hook) { put_hook_ = std::move(hook); }
  bool put(int peer, uint32_t remote_key, uint64_t remote_off, const void* src, uint64_t bytes) override;
  bool signal(int peer, uint32_t slot, uint64_t add) override;
  void shutdown();
  uint64_t bytesSent() const override { return bytes_sent_.load(); }
  uint64_t bytesReceived() const override { return bytes_recv_.load(); }
  void setAdvertisedHost(const std::string& h) { host_ = h; }

 private:
  struct Conn { int fd = -1; std::mutex mu; };
  struct Region { char* ptr; size_t bytes; };
  void acceptLoop();
  void readerLoop(int fd);

  std::string host_ = "127.0.0.1";
  int port_ = 0;
  int listen_fd_ = -1;
  std::atomic<bool> running_{false};
  std::thread accept_thread_;
  std::mutex mu_;
  std::vector<std::thread> readers_;
  std::vector<int> reader_fds_;
  std::map<int, std::string> endpoints_;
  std::map<int, std::shared_ptr<Conn>> conns_;
  std::vector<Region> regions_;
  std::function<void(uint32_t, uint64_t, uint64_t)> put_hook_;
  std::atomic<uint64_t>* signals_ = nullptr;
  uint32_t num_signals_ = 0;
  std::atomic<uint64_t> bytes_sent_{0}, bytes_recv_{0};
};

}  // namespace pccl
