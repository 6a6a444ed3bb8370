#include "bootstrap/hub.h"
#include <poll.h>
#include <time.h>
#include <unistd.h>
#include <cstring>
#include <algorithm>
#include <fstream>
#include <sstream>
#include "bootstrap/socket.h"
#include "common/env.h"
#include "common/json.h"
#include "common/log.h"

namespace hcclb {

namespace {
struct FrameHdr { uint32_t magic, type, key_len, payload_len, nmembers, member; };
struct ReplyHdr { uint32_t magic, status, total_len; };
uint64_t now_ms()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}
constexpr uint32_t kMaxFrame = 64u << 20;
}  // namespace

Hub *Hub::start(const std::string &ip, int port, int family, std::string *err)
{
    Hub *h = new Hub();
    h->port_ = port;
    h->ip_ = ip;
    h->lfd_ = net::tcp_listen(family == 6 ? "::" : "0.0.0.0", &h->port_, family);
    if (h->lfd_ < 0 || pipe(h->wake_) != 0) {
        if (err) *err = "cannot listen on port " + std::to_string(port);
        delete h;
        return nullptr;
    }
    // connection whitelist (reference: framework/common/src/topo/hccl_whitelist.cc: JSON file with a "host_ip" array, enabled
    // by HCCL_WHITELIST_DISABLE=0): a hub that cannot load its list refuses to start rather than run open
    const EnvConfig &env = env_config();
    if (env.whitelist_enable) {
        std::ifstream f(env.whitelist_file);
        std::stringstream ss;
        ss << f.rdbuf();
        JsonValue v;
        std::string jerr;
        const JsonValue *ips = nullptr;
        if (!f || !json_parse(ss.str(), &v, &jerr) || !(ips = v.get("host_ip")) || ips->type != JsonValue::ARR) {
            if (err) *err = "whitelist file " + env.whitelist_file + " cannot be read as {\"host_ip\": [...]}" + (jerr.empty() ? "" : ": " + jerr);
            delete h;
            return nullptr;
        }
        for (const JsonValue &ipv : ips->arr)
            if (ipv.type == JsonValue::STR) h->whitelist_.push_back(ipv.str);
        h->whitelist_on_ = true;
    }
    h->th_ = std::thread([h] { h->run(); });
    return h;
}

Hub::~Hub() { stop(); }

void Hub::stop()
{
    if (stop_.exchange(true)) return;
    if (wake_[1] >= 0) { char c = 1; (void)!write(wake_[1], &c, 1); }
    if (th_.joinable()) th_.join();
    for (int fd : clients_) net::close_fd(fd);
    clients_.clear();
    net::close_fd(lfd_);
    net::close_fd(wake_[0]);
    net::close_fd(wake_[1]);
    lfd_ = wake_[0] = wake_[1] = -1;
}

void Hub::drop_client(int fd)
{
    for (size_t i = 0; i < clients_.size(); ++i)
        if (clients_[i] == fd) { clients_.erase(clients_.begin() + i); break; }
    net::close_fd(fd);
}

bool Hub::handle_frame(int fd)
{
    FrameHdr h;
    if (!net::recv_all(fd, &h, sizeof(h), 5000)) return false;
    if (h.magic != kHubMagic || h.key_len > 4096 || h.payload_len > kMaxFrame) return false;
    std::string key(h.key_len, 0), payload(h.payload_len, 0);
    if (h.key_len && !net::recv_all(fd, &key[0], h.key_len, 5000)) return false;
    if (h.payload_len && !net::recv_all(fd, &payload[0], h.payload_len, 30000)) return false;
    if (h.type == HUB_BYE) return false;
    if (h.type == HUB_RENDEZVOUS) {
        if (h.nmembers == 0 || h.nmembers > 4096 || h.member >= h.nmembers) return false;
        Pending &p = pending_[key];
        if (p.fds.empty()) {
            p.nmembers = h.nmembers;
            p.fds.assign(h.nmembers, -1);
            p.payloads.assign(h.nmembers, std::string());
            p.have.assign(h.nmembers, false);
            p.count = 0;
        }
        uint32_t status = HCCL_SUCCESS;
        if (p.nmembers != h.nmembers || p.have[h.member]) status = HCCL_E_PARA;  // inconsistent group description
        if (status != HCCL_SUCCESS) {
            ReplyHdr r{kHubMagic, status, 0};
            net::send_all(fd, &r, sizeof(r));
            return true;
        }
        p.fds[h.member] = fd;
        p.payloads[h.member] = std::move(payload);
        p.have[h.member] = true;
        if (++p.count == p.nmembers) {
            std::string body;
            for (auto &pl : p.payloads) {
                uint32_t l = (uint32_t)pl.size();
                body.append((const char *)&l, 4);
                body.append(pl);
            }
            ReplyHdr r{kHubMagic, HCCL_SUCCESS, (uint32_t)body.size()};
            for (int cfd : p.fds) {
                net::send_all(cfd, &r, sizeof(r));
                net::send_all(cfd, body.data(), body.size());
            }
            pending_.erase(key);
        }
        return true;
    }
    if (h.type == HUB_HEARTBEAT) {
        if (payload.size() != sizeof(HeartbeatMsg)) return false;
        HeartbeatMsg m;
        memcpy(&m, payload.data(), sizeof(m));
        if (m.rank >= 16 || m.nranks > 16) return false;
        auto &grp = beats_[key];
        grp[m.rank] = Beat{now_ms(), m};
        HeartbeatSummary s;
        memset(&s, 0, sizeof(s));
        s.first_bad_rank = 0xffffffffu;
        uint64_t now = now_ms();
        for (uint32_t r = 0; r < m.nranks; ++r) {
            auto it = grp.find(r);
            if (it == grp.end()) continue;  // not yet registered: unknown, not lost
            uint32_t st = it->second.msg.status;
            if (st == PEER_OK && now - it->second.last_ms > it->second.msg.lost_ms) st = PEER_LOST;
            s.status[r] = st;
            s.error_code[r] = it->second.msg.error_code;
            s.epoch[r] = it->second.msg.epoch;
            if (st != PEER_OK && s.first_bad_rank == 0xffffffffu) s.first_bad_rank = r;
        }
        ReplyHdr r{kHubMagic, HCCL_SUCCESS, (uint32_t)sizeof(s)};
        return net::send_all(fd, &r, sizeof(r)) && net::send_all(fd, &s, sizeof(s));
    }
    return false;
}

void Hub::run()
{
    while (!stop_.load()) {
        std::vector<pollfd> pf;
        pf.push_back({lfd_, POLLIN, 0});
        pf.push_back({wake_[0], POLLIN, 0});
        for (int fd : clients_) pf.push_back({fd, POLLIN, 0});
        int rc = poll(pf.data(), pf.size(), 500);
        if (rc <= 0) continue;
        if (pf[1].revents) break;
        if (pf[0].revents & POLLIN) {
            int fd = net::accept_timeout(lfd_, 0);
            if (fd >= 0 && whitelist_on_) {
                std::string peer = net::peer_address(fd);
                if (std::find(whitelist_.begin(), whitelist_.end(), peer) == whitelist_.end()) {
                    HLOG_ERROR("connection from %s refused: address not in the whitelist", peer.c_str());
                    net::close_fd(fd);
                    fd = -1;
                }
            }
            if (fd >= 0) clients_.push_back(fd);
        }
        for (size_t i = 2; i < pf.size(); ++i) {
            if (!(pf[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
            if (!handle_frame(pf[i].fd)) drop_client(pf[i].fd);
        }
    }
}

HubClient::~HubClient()
{
    bye();
}
void HubClient::bye()
{
    std::lock_guard<std::mutex> lk(mu_);
    if (fd_ < 0) return;
    FrameHdr h{kHubMagic, HUB_BYE, 0, 0, 0, 0};
    net::send_all(fd_, &h, sizeof(h));
    net::close_fd(fd_);
    fd_ = -1;
}
HcclResult HubClient::connect(const std::string &ip, int port, int family, int timeout_ms)
{
    fd_ = net::tcp_connect(ip, port, timeout_ms, family);
    if (fd_ < 0) {
        HLOG_ERROR("cannot reach bootstrap hub %s:%d within %d ms", ip.c_str(), port, timeout_ms);
        return HCCL_E_TCP_CONNECT;
    }
    return HCCL_SUCCESS;
}

static HcclResult transact(int fd, uint32_t type, const std::string &key, uint32_t nmembers, uint32_t member,
                           const std::string &payload, std::string *body, int timeout_ms)
{
    if (fd < 0) return HCCL_E_TCP_CONNECT;
    FrameHdr h{kHubMagic, type, (uint32_t)key.size(), (uint32_t)payload.size(), nmembers, member};
    if (!net::send_all(fd, &h, sizeof(h)) || !net::send_all(fd, key.data(), key.size()) ||
        !net::send_all(fd, payload.data(), payload.size()))
        return HCCL_E_TCP_TRANSFER;
    ReplyHdr r;
    if (!net::recv_all(fd, &r, sizeof(r), timeout_ms)) return HCCL_E_TIMEOUT;
    if (r.magic != kHubMagic || r.total_len > kMaxFrame) return HCCL_E_TCP_TRANSFER;
    if (r.status != HCCL_SUCCESS) return (HcclResult)r.status;
    body->assign(r.total_len, 0);
    if (r.total_len && !net::recv_all(fd, &(*body)[0], r.total_len, timeout_ms)) return HCCL_E_TCP_TRANSFER;
    return HCCL_SUCCESS;
}

HcclResult HubClient::rendezvous(const std::string &key, uint32_t nmembers, uint32_t member, const std::string &payload,
                                 std::vector<std::string> *out, int timeout_ms)
{
    std::lock_guard<std::mutex> lk(mu_);
    std::string body;
    HcclResult rc = transact(fd_, HUB_RENDEZVOUS, key, nmembers, member, payload, &body, timeout_ms);
    if (rc != HCCL_SUCCESS) {
        HLOG_ERROR("rendezvous '%s' (%u members) failed: %d", key.c_str(), nmembers, (int)rc);
        return rc;
    }
    if (out) {
        out->clear();
        size_t pos = 0;
        for (uint32_t i = 0; i < nmembers; ++i) {
            if (pos + 4 > body.size()) return HCCL_E_TCP_TRANSFER;
            uint32_t l;
            memcpy(&l, body.data() + pos, 4);
            pos += 4;
            if (pos + l > body.size()) return HCCL_E_TCP_TRANSFER;
            out->emplace_back(body.data() + pos, l);
            pos += l;
        }
    }
    return HCCL_SUCCESS;
}
HcclResult HubClient::barrier(const std::string &key, uint32_t nmembers, uint32_t member, int timeout_ms)
{
    return rendezvous(key, nmembers, member, std::string(), nullptr, timeout_ms);
}
HcclResult HubClient::heartbeat(const std::string &group, const HeartbeatMsg &msg, HeartbeatSummary *sum, int timeout_ms)
{
    std::lock_guard<std::mutex> lk(mu_);
    std::string body, payload((const char *)&msg, sizeof(msg));
    HcclResult rc = transact(fd_, HUB_HEARTBEAT, group, 0, 0, payload, &body, timeout_ms);
    if (rc != HCCL_SUCCESS) return rc;
    if (body.size() != sizeof(HeartbeatSummary)) return HCCL_E_TCP_TRANSFER;
    memcpy(sum, body.data(), sizeof(*sum));
    return HCCL_SUCCESS;
}

}  // namespace hcclb
