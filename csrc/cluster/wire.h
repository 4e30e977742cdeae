// Socket helpers and length-prefixed framing for the control plane and the TCP data plane.
// The reference reads up to 4096 bytes and parses whatever arrived as one JSON document
// (csrc/cluster/daemon.cc:215-243), which breaks as soon as two messages coalesce or one is split;
// every message here is [magic u32][kind u32][length u64][payload].
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace pccl {
namespace wire {

constexpr uint32_t kMagic = 0x5043434cu;   // "PCCL"
constexpr uint64_t kMaxFrame = 1ull << 32;

struct FrameHeader {
  uint32_t magic;
  uint32_t kind;
  uint64_t length;
};

// Listens on host:port (port 0 = ephemeral; *port receives the bound port).  Returns fd or -1.
int tcpListen(const std::string& host, int* port, int backlog = 128);
// Connects with retry until timeout_ms elapses.  Returns fd or -1.
int tcpConnect(const std::string& host, int port, int timeout_ms);
int acceptOne(int listen_fd, int timeout_ms);   // -1 on timeout/error
void closeFd(int fd);
void shutdownFd(int fd);

bool sendAll(int fd, const void* data, size_t n);
bool recvAll(int fd, void* data, size_t n);   // false on EOF or error
bool sendFrame(int fd, uint32_t kind, const void* payload, uint64_t n);
bool sendFrame2(int fd, uint32_t kind, const void* head, uint64_t nh, const void* body, uint64_t nb);
bool recvHeader(int fd, FrameHeader* h);
bool recvFrame(int fd, uint32_t* kind, std::string* payload);

bool splitHostPort(const std::string& endpoint, std::string* host, int* port);

// AF_UNIX (abstract namespace) helpers with file-descriptor passing, used to hand CUDA VMM
// handles to peer processes of the same host.
int unixListen(const std::string& abstract_name);
int unixConnect(const std::string& abstract_name, int timeout_ms);
bool sendFd(int sock, int fd_to_send, uint64_t tag);
bool recvFd(int sock, int* fd_out, uint64_t* tag);
long peerUid(int sock);      // user id of the process at the other end of an AF_UNIX socket (SO_PEERCRED); -1 if unknown

}  // namespace wire
}  // namespace pccl
