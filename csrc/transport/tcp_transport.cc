#include "tcp_transport.h"

#include <dlfcn.h>

#include <cstring>
#include <stdexcept>

#include "../cluster/wire.h"
#include "../common/env.h"
#include "../common/log.h"

namespace pccl {

namespace {
constexpr uint32_t kPut = 10, kSignal = 11;
struct PutHead { uint32_t key; uint32_t pad; uint64_t off; };
struct SigHead { uint32_t slot; uint32_t pad; uint64_t add; };
}  // namespace

TcpTransport::~TcpTransport() { shutdown(); }

std::string TcpTransport::activate() {
  if (!running_.load()) {
    port_ = 0;
    listen_fd_ = wire::tcpListen("0.0.0.0", &port_);
    if (listen_fd_ < 0) throw std::runtime_error("tcp transport: cannot open a listening socket");
    running_.store(true);
    accept_thread_ = std::thread([this] { acceptLoop(); });
  }
  return host_ + ":" + std::to_string(port_);
}

void TcpTransport::shutdown() {
  if (!running_.exchange(false)) return;
  wire::shutdownFd(listen_fd_);
  if (accept_thread_.joinable()) accept_thread_.join();
  std::vector<std::thread> readers;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : conns_) wire::shutdownFd(kv.second->fd);
    for (int fd : reader_fds_) wire::shutdownFd(fd);
    readers.swap(readers_);
  }
  for (auto& t : readers)
    if (t.joinable()) t.join();
  std::lock_guard<std::mutex> g(mu_);
  for (auto& kv : conns_) wire::closeFd(kv.second->fd);
  for (int fd : reader_fds_) wire::closeFd(fd);
  conns_.clear();
  reader_fds_.clear();
  wire::closeFd(listen_fd_);
  listen_fd_ = -1;
}

uint32_t TcpTransport::regBuffer(void* ptr, size_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  regions_.push_back(Region{static_cast<char*>(ptr), bytes});
  return static_cast<uint32_t>(regions_.size() - 1);
}

void TcpTransport::unregBuffer(uint32_t key) {
  std::lock_guard<std::mutex> g(mu_);
  if (key < regions_.size()) regions_[key] = Region{nullptr, 0};
}

void TcpTransport::regRemoteHandle(int peer, const std::string& endpoint) {
  std::lock_guard<std::mutex> g(mu_);
  endpoints_[peer] = endpoint;
}

void TcpTransport::connect(int peer) {
  std::string ep;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (conns_.count(peer)) return;
    auto it = endpoints_.find(peer);
    if (it == endpoints_.end()) throw std::runtime_error("tcp transport: no endpoint known for peer " + std::to_string(peer));
    ep = it->second;
  }
  std::string host;
  int port = 0;
  if (!wire::splitHostPort(ep, &host, &port)) throw std::runtime_error("tcp transport: bad endpoint " + ep);
  int fd = wire::tcpConnect(host, port, 30000);
  if (fd < 0) throw std::runtime_error("tcp transport: cannot connect to " + ep);
  auto c = std::make_shared<Conn>();
  c->fd = fd;
  std::lock_guard<std::mutex> g(mu_);
  conns_[peer] = c;
}

void TcpTransport::disconnect(int peer) {
  std::shared_ptr<Conn> c;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = conns_.find(peer);
    if (it == conns_.end()) return;
    c = it->second;
    conns_.erase(it);
  }
  std::lock_guard<std::mutex> g(c->mu);
  wire::shutdownFd(c->fd);
  wire::closeFd(c->fd);
  c->fd = -1;
}

bool TcpTransport::put(int peer, uint32_t key, uint64_t off, const void* src, uint64_t bytes) {
  std::shared_ptr<Conn> c;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = conns_.find(peer);
    if (it == conns_.end()) return false;
    c = it->second;
  }
  PutHead h{key, 0, off};
  std::lock_guard<std::mutex> g(c->mu);
  if (c->fd < 0) return false;
  bool ok = wire::sendFrame2(c->fd, kPut, &h, sizeof(h), src, bytes);
  if (ok) bytes_sent_.fetch_add(bytes);
  return ok;
}

bool TcpTransport::signal(int peer, uint32_t slot, uint64_t add) {
  std::shared_ptr<Conn> c;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = conns_.find(peer);
    if (it == conns_.end()) return false;
    c = it->second;
  }
  SigHead h{slot, 0, add};
  std::lock_guard<std::mutex> g(c->mu);
  if (c->fd < 0) return false;
  return wire::sendFrame(c->fd, kSignal, &h, sizeof(h));
}

void TcpTransport::acceptLoop() {
  while (running_.load()) {
    int fd = wire::acceptOne(listen_fd_, 100);
    if (fd < 0) continue;
    std::lock_guard<std::mutex> g(mu_);
    reader_fds_.push_back(fd);
    readers_.emplace_back([this, fd] { readerLoop(fd); });
  }
}

void TcpTransport::readerLoop(int fd) {
  std::vector<char> sink;
  while (running_.load()) {
    wire::FrameHeader h;
    if (!wire::recvHeader(fd, &h)) break;
    if (h.kind == kPut && h.length >= sizeof(PutHead)) {
      PutHead ph;
      if (!wire::recvAll(fd, &ph, sizeof(ph))) break;
      uint64_t n = h.length - sizeof(ph);
      char* dst = nullptr;
      {
        std::lock_guard<std::mutex> g(mu_);
        if (ph.key < regions_.size() && regions_[ph.key].ptr && ph.off <= regions_[ph.key].bytes &&
            n <= regions_[ph.key].bytes - ph.off)
          dst = regions_[ph.key].ptr + ph.off;
      }
      if (!dst) {   // out-of-range write: drain and drop, never touch memory
        PCCL_LOG_ERROR("tcp transport: dropping PUT outside registered buffer (key %u off %llu len %llu)", ph.key,
                       static_cast<unsigned long long>(ph.off), static_cast<unsigned long long>(n));
        sink.resize(n);
        dst = sink.data();
      }
      const bool real = dst != sink.data() || n == 0;
      if (n && !wire::recvAll(fd, dst, n)) break;
      bytes_recv_.fetch_add(n);
      if (real && n && put_hook_) put_hook_(ph.key, ph.off, n);
    } else if (h.kind == kSignal && h.length == sizeof(SigHead)) {
      SigHead sh;
      if (!wire::recvAll(fd, &sh, sizeof(sh))) break;
      if (signals_ && sh.slot < num_signals_) signals_[sh.slot].fetch_add(sh.add, std::memory_order_release);
    } else {
      sink.resize(h.length);
      if (h.length && !wire::recvAll(fd, sink.data(), h.length)) break;
    }
  }
}

}  // namespace pccl
