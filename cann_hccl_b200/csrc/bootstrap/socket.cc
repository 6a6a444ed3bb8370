#include "bootstrap/socket.h"
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>
#include <cstring>
#include "common/log.h"

namespace hcclb {
namespace net {

static uint64_t now_ms()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

static bool fill_addr(const std::string &ip, int port, int family, sockaddr_storage *ss, socklen_t *len)
{
    memset(ss, 0, sizeof(*ss));
    if (family == 6) {
        auto *a = (sockaddr_in6 *)ss;
        a->sin6_family = AF_INET6;
        a->sin6_port = htons((uint16_t)port);
        if (inet_pton(AF_INET6, ip.empty() ? "::" : ip.c_str(), &a->sin6_addr) != 1) return false;
        *len = sizeof(*a);
    } else {
        auto *a = (sockaddr_in *)ss;
        a->sin_family = AF_INET;
        a->sin_port = htons((uint16_t)port);
        if (inet_pton(AF_INET, ip.empty() ? "0.0.0.0" : ip.c_str(), &a->sin_addr) != 1) return false;
        *len = sizeof(*a);
    }
    return true;
}

int tcp_listen(const std::string &ip, int *port, int family)
{
    sockaddr_storage ss;
    socklen_t len;
    if (!fill_addr(ip, *port, family, &ss, &len)) return -1;
    int fd = socket(family == 6 ? AF_INET6 : AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (bind(fd, (sockaddr *)&ss, len) != 0 || listen(fd, 256) != 0) {
        close(fd);
        return -1;
    }
    sockaddr_storage got;
    socklen_t glen = sizeof(got);
    if (getsockname(fd, (sockaddr *)&got, &glen) == 0)
        *port = ntohs(family == 6 ? ((sockaddr_in6 *)&got)->sin6_port : ((sockaddr_in *)&got)->sin_port);
    return fd;
}

int tcp_connect(const std::string &ip, int port, int timeout_ms, int family)
{
    sockaddr_storage ss;
    socklen_t len;
    if (!fill_addr(ip, port, family, &ss, &len)) return -1;
    uint64_t deadline = now_ms() + (uint64_t)timeout_ms;
    for (;;) {
        int fd = socket(family == 6 ? AF_INET6 : AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd < 0) return -1;
        if (connect(fd, (sockaddr *)&ss, len) == 0) {
            int one = 1;
            setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            return fd;
        }
        close(fd);
        if (now_ms() >= deadline) return -1;
        usleep(20000);
    }
}

int accept_timeout(int lfd, int timeout_ms)
{
    pollfd p{lfd, POLLIN, 0};
    int rc = poll(&p, 1, timeout_ms);
    if (rc == 0) return -2;
    if (rc < 0) return -1;
    int fd = accept4(lfd, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd >= 0) {
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    }
    return fd;
}

std::string peer_address(int fd)
{
    sockaddr_storage ss;
    socklen_t len = sizeof(ss);
    if (getpeername(fd, (sockaddr *)&ss, &len) != 0) return "";
    char buf[INET6_ADDRSTRLEN] = {0};
    if (ss.ss_family == AF_INET) inet_ntop(AF_INET, &((sockaddr_in *)&ss)->sin_addr, buf, sizeof(buf));
    else if (ss.ss_family == AF_INET6) inet_ntop(AF_INET6, &((sockaddr_in6 *)&ss)->sin6_addr, buf, sizeof(buf));
    std::string a(buf);
    if (a.rfind("::ffff:", 0) == 0) a = a.substr(7);
    return a;
}

bool send_all(int fd, const void *buf, size_t len)
{
    const char *p = (const char *)buf;
    while (len) {
        ssize_t n = send(fd, p, len, MSG_NOSIGNAL);
        if (n < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += n;
        len -= (size_t)n;
    }
    return true;
}

bool recv_all(int fd, void *buf, size_t len, int timeout_ms)
{
    char *p = (char *)buf;
    uint64_t deadline = timeout_ms < 0 ? 0 : now_ms() + (uint64_t)timeout_ms;
    while (len) {
        if (timeout_ms >= 0) {
            uint64_t now = now_ms();
            if (now >= deadline) return false;
            pollfd pf{fd, POLLIN, 0};
            int rc = poll(&pf, 1, (int)(deadline - now));
            if (rc == 0) return false;
            if (rc < 0) {
                if (errno == EINTR) continue;
                return false;
            }
        }
        ssize_t n = recv(fd, p, len, 0);
        if (n == 0) return false;
        if (n < 0) {
            if (errno == EINTR) continue;
            return false;
        }
        p += n;
        len -= (size_t)n;
    }
    return true;
}

void close_fd(int fd)
{
    if (fd >= 0) close(fd);
}

static socklen_t unix_addr(const std::string &name, sockaddr_un *a)
{
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    size_t n = name.size() < sizeof(a->sun_path) - 2 ? name.size() : sizeof(a->sun_path) - 2;
    memcpy(a->sun_path + 1, name.data(), n);  // leading NUL = abstract namespace
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}
int unix_listen(const std::string &name)
{
    sockaddr_un a;
    socklen_t len = unix_addr(name, &a);
    int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return -1;
    if (bind(fd, (sockaddr *)&a, len) != 0 || listen(fd, 64) != 0) {
        close(fd);
        return -1;
    }
    return fd;
}
int unix_connect(const std::string &name, int timeout_ms)
{
    sockaddr_un a;
    socklen_t len = unix_addr(name, &a);
    uint64_t deadline = now_ms() + (uint64_t)timeout_ms;
    for (;;) {
        int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd < 0) return -1;
        if (connect(fd, (sockaddr *)&a, len) == 0) return fd;
        close(fd);
        if (now_ms() >= deadline) return -1;
        usleep(10000);
    }
}
bool send_fds(int sock, int src_rank, const int *fds, int nfds)
{
    int32_t head[2] = {src_rank, nfds};
    msghdr msg;
    memset(&msg, 0, sizeof(msg));
    iovec iov{head, sizeof(head)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int) * 16)];
    if (nfds > 16) return false;
    if (nfds > 0) {
        memset(ctrl, 0, sizeof(ctrl));
        msg.msg_control = ctrl;
        msg.msg_controllen = CMSG_SPACE(sizeof(int) * nfds);
        cmsghdr *c = CMSG_FIRSTHDR(&msg);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int) * nfds);
        memcpy(CMSG_DATA(c), fds, sizeof(int) * nfds);
    }
    return sendmsg(sock, &msg, MSG_NOSIGNAL) == (ssize_t)sizeof(head);
}
bool recv_fds(int sock, int *src_rank, std::vector<int> *fds, int timeout_ms)
{
    pollfd pf{sock, POLLIN, 0};
    if (poll(&pf, 1, timeout_ms) <= 0) return false;
    int32_t head[2] = {0, 0};
    msghdr msg;
    memset(&msg, 0, sizeof(msg));
    iovec iov{head, sizeof(head)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int) * 16)];
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    if (recvmsg(sock, &msg, MSG_CMSG_CLOEXEC) != (ssize_t)sizeof(head)) return false;
    *src_rank = head[0];
    fds->clear();
    for (cmsghdr *c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
        if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
            int n = (int)((c->cmsg_len - CMSG_LEN(0)) / sizeof(int));
            for (int i = 0; i < n; ++i) {
                int fd;
                memcpy(&fd, CMSG_DATA(c) + i * sizeof(int), sizeof(int));
                fds->push_back(fd);
            }
        }
    }
    return (int)fds->size() == head[1];
}

std::string local_ip()
{
    std::string out = "127.0.0.1";
    ifaddrs *ifa = nullptr;
    if (getifaddrs(&ifa) != 0) return out;
    for (ifaddrs *i = ifa; i; i = i->ifa_next) {
        if (!i->ifa_addr || i->ifa_addr->sa_family != AF_INET) continue;
        auto *a = (sockaddr_in *)i->ifa_addr;
        if (ntohl(a->sin_addr.s_addr) >> 24 == 127) continue;
        char buf[64];
        if (inet_ntop(AF_INET, &a->sin_addr, buf, sizeof(buf))) {
            out = buf;
            break;
        }
    }
    freeifaddrs(ifa);
    return out;
}

}  // namespace net
}  // namespace hcclb
