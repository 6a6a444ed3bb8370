// Small blocking-socket helpers used by the bootstrap hub, heartbeat and handle exchange.
#pragma once
#include <string>
#include <vector>
#include "hccl/hccl_types.h"
namespace hcclb {
namespace net {
// Listen on ip:port (port 0 = pick one; the chosen port is returned through *port). Returns fd or -1.
int tcp_listen(const std::string &ip, int *port, int family = 4);
// Connect with retries until timeout_ms elapses. Returns fd or -1.
int tcp_connect(const std::string &ip, int port, int timeout_ms, int family = 4);
// Accept with a bound; returns fd, -1 on error, -2 on timeout.
int accept_timeout(int lfd, int timeout_ms);
// Numeric address of the peer of a connected TCP socket ("" when unknown); IPv4-mapped IPv6 addresses come back as IPv4.
std::string peer_address(int fd);
bool send_all(int fd, const void *buf, size_t len);
// Receive exactly len bytes; timeout_ms < 0 waits forever. Returns false on error / EOF / timeout.
bool recv_all(int fd, void *buf, size_t len, int timeout_ms = -1);
void close_fd(int fd);
// Unix-domain sockets in the abstract namespace, used to pass file descriptors (SCM_RIGHTS) between ranks of a node.
int unix_listen(const std::string &name);
int unix_connect(const std::string &name, int timeout_ms);
bool send_fds(int sock, int src_rank, const int *fds, int nfds);
bool recv_fds(int sock, int *src_rank, std::vector<int> *fds, int timeout_ms);
// First non-loopback IPv4 address of this host, or 127.0.0.1.
std::string local_ip();
}  // namespace net
}  // namespace hcclb
