#include "wire.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <thread>

namespace pccl {
namespace wire {

static void tune(int fd) {
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int buf = 4 << 20;
  ::setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  ::setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

static bool resolve(const std::string& host, int port, sockaddr_in* out) {
  std::memset(out, 0, sizeof(*out));
  out->sin_family = AF_INET;
  out->sin_port = htons(static_cast<uint16_t>(port));
  std::string h = host.empty() ? "0.0.0.0" : host;
  if (h == "localhost") h = "127.0.0.1";
  if (::inet_pton(AF_INET, h.c_str(), &out->sin_addr) == 1) return true;
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  if (::getaddrinfo(h.c_str(), nullptr, &hints, &res) != 0 || !res) return false;
  out->sin_addr = reinterpret_cast<sockaddr_in*>(res->ai_addr)->sin_addr;
  ::freeaddrinfo(res);
  return true;
}

int tcpListen(const std::string& host, int* port, int backlog) {
  sockaddr_in addr;
  if (!resolve(host, port ? *port : 0, &addr)) return -1;
  int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  int one = 1;
  ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd, backlog) != 0) {
    ::close(fd);
    return -1;
  }
  socklen_t len = sizeof(addr);
  if (port && ::getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len) == 0) *port = ntohs(addr.sin_port);
  return fd;
}

int tcpConnect(const std::string& host, int port, int timeout_ms) {
  sockaddr_in addr;
  if (!resolve(host.empty() ? "127.0.0.1" : host, port, &addr)) return -1;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
      tune(fd);
      return fd;
    }
    ::close(fd);
    if (std::chrono::steady_clock::now() >= deadline) return -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}

int acceptOne(int listen_fd, int timeout_ms) {
  pollfd p{listen_fd, POLLIN, 0};
  int r = ::poll(&p, 1, timeout_ms);
  if (r <= 0 || !(p.revents & POLLIN)) return -1;
  int fd = ::accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
  if (fd >= 0) tune(fd);
  return fd;
}

void closeFd(int fd) { if (fd >= 0) ::close(fd); }
void shutdownFd(int fd) { if (fd >= 0) ::shutdown(fd, SHUT_RDWR); }

bool sendAll(int fd, const void* data, size_t n) {
  const char* p = static_cast<const char*>(data);
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}

bool recvAll(int fd, void* data, size_t n) {
  char* p = static_cast<char*>(data);
  while (n) {
    ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

bool sendFrame(int fd, uint32_t kind, const void* payload, uint64_t n) {
  return sendFrame2(fd, kind, payload, n, nullptr, 0);
}

bool sendFrame2(int fd, uint32_t kind, const void* head, uint64_t nh, const void* body, uint64_t nb) {
  FrameHeader h{kMagic, kind, nh + nb};
  if (!sendAll(fd, &h, sizeof(h))) return false;
  if (nh && !sendAll(fd, head, nh)) return false;
  if (nb && !sendAll(fd, body, nb)) return false;
  return true;
}

bool recvHeader(int fd, FrameHeader* h) {
  if (!recvAll(fd, h, sizeof(*h))) return false;
  return h->magic == kMagic && h->length <= kMaxFrame;
}

bool recvFrame(int fd, uint32_t* kind, std::string* payload) {
  FrameHeader h;
  if (!recvHeader(fd, &h)) return false;
  payload->resize(h.length);
  if (h.length && !recvAll(fd, payload->data(), h.length)) return false;
  *kind = h.kind;
  return true;
}

bool splitHostPort(const std::string& ep, std::string* host, int* port) {
  size_t c = ep.rfind(':');
  if (c == std::string::npos) return false;
  *host = ep.substr(0, c);
  char* end = nullptr;
  long v = std::strtol(ep.c_str() + c + 1, &end, 10);
  if (!end || *end != '\0' || v < 0 || v > 65535) return false;
  *port = static_cast<int>(v);
  return true;
}

static socklen_t abstractAddr(const std::string& name, sockaddr_un* a) {
  std::memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  size_t n = std::min(name.size(), sizeof(a->sun_path) - 2);
  std::memcpy(a->sun_path + 1, name.data(), n);   // leading NUL = abstract namespace
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int unixListen(const std::string& name) {
  int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  sockaddr_un a;
  socklen_t len = abstractAddr(name, &a);
  if (::bind(fd, reinterpret_cast<sockaddr*>(&a), len) != 0 || ::listen(fd, 64) != 0) {
    ::close(fd);
    return -1;
  }
  return fd;
}

int unixConnect(const std::string& name, int timeout_ms) {
  sockaddr_un a;
  socklen_t len = abstractAddr(name, &a);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    if (::connect(fd, reinterpret_cast<sockaddr*>(&a), len) == 0) return fd;
    ::close(fd);
    if (std::chrono::steady_clock::now() >= deadline) return -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}

bool sendFd(int sock, int fd_to_send, uint64_t tag) {
  msghdr msg{};
  iovec iov{&tag, sizeof(tag)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  std::memset(ctrl, 0, sizeof(ctrl));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  if (fd_to_send >= 0) {
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd_to_send, sizeof(int));
  }
  return ::sendmsg(sock, &msg, MSG_NOSIGNAL) == static_cast<ssize_t>(sizeof(tag));
}

bool recvFd(int sock, int* fd_out, uint64_t* tag) {
  msghdr msg{};
  uint64_t t = 0;
  iovec iov{&t, sizeof(t)};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t r = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
  if (r != static_cast<ssize_t>(sizeof(t))) return false;
  *fd_out = -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c))
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) std::memcpy(fd_out, CMSG_DATA(c), sizeof(int));
  if (tag) *tag = t;
  return true;
}

long peerUid(int sock) {
  ucred cr{};
  socklen_t len = sizeof(cr);
  if (::getsockopt(sock, SOL_SOCKET, SO_PEERCRED, &cr, &len) != 0 || len != sizeof(cr)) return -1;
  return static_cast<long>(cr.uid);
}

}  // namespace wire
}  // namespace pccl
