// Bootstrap hub: the TCP rendezvous point started by HcclGetRootInfo on the root rank, and its client.
// It plays the role of the reference's TopoInfoExchangeServer / TopoInfoExchangeAgent pair
// (framework/common/src/topo/topoinfo_exchange_server.cc:43-80, topoinfo_exchange_agent.cc) and, because it
// stays alive for the communicator's lifetime, also carries the control traffic that the reference sends
// over separate sockets: memory-handle exchange, heartbeat status, retry agreement, sub-communicator setup.
//
// Protocol: a client sends frames {magic,type,key_len,payload_len,nmembers,member}+key+payload.
//  - RENDEZVOUS: the hub holds the frame until `nmembers` frames with the same key arrived, then answers each
//    member with all payloads in member order (an all-gather keyed by name; any subset of ranks may meet).
//  - HEARTBEAT: payload = HeartbeatMsg; the hub records it and answers with a HeartbeatSummary of the group.
//  - BYE: the client leaves.
#pragma once
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include "hccl/hccl_types.h"

namespace hcclb {

constexpr uint32_t kHubMagic = 0x48434c42u;  // "HCLB"
enum HubFrameType : uint32_t { HUB_RENDEZVOUS = 1, HUB_HEARTBEAT = 2, HUB_BYE = 3 };

enum PeerHealth : uint32_t { PEER_OK = 0, PEER_LOST = 1, PEER_ERROR = 2, PEER_STUCK = 3 };

struct HeartbeatMsg {
    uint32_t rank, nranks;
    uint32_t status;      // PeerHealth the rank reports about itself
    uint32_t error_code;  // HcclResult when status == PEER_ERROR
    uint64_t head, tail;  // op-execution counters
    uint32_t lost_ms;     // silence after which the hub declares this group's members lost
    uint32_t epoch;       // number of resumes the rank has gone through; older reports are stale
};
struct HeartbeatSummary {
    uint32_t status[16];      // per rank PeerHealth as the hub sees it
    uint32_t error_code[16];  // per rank last reported error
    uint32_t epoch[16];       // per rank resume epoch of that report
    uint32_t first_bad_rank;  // 0xffffffff when all fine
    uint32_t pad;
};

class Hub {
public:
    // Start listening on ip:port (port 0 picks a free one) and run the service thread.
    static Hub *start(const std::string &ip, int port, int family, std::string *err);
    ~Hub();
    int port() const { return port_; }
    const std::string &ip() const { return ip_; }
    void stop();

private:
    Hub() = default;
    void run();
    struct Pending { uint32_t nmembers; std::vector<int> fds; std::vector<std::string> payloads; std::vector<bool> have; uint32_t count; };
    struct Beat { uint64_t last_ms; HeartbeatMsg msg; };
    bool handle_frame(int fd);
    void drop_client(int fd);
    int lfd_ = -1, port_ = 0, wake_[2] = {-1, -1};
    std::string ip_;
    std::thread th_;
    std::atomic<bool> stop_{false};
    std::vector<int> clients_;
    bool whitelist_on_ = false;              // HCCL_WHITELIST_DISABLE=0: only the listed addresses may connect
    std::vector<std::string> whitelist_;     // numeric addresses from HCCL_WHITELIST_FILE ("host_ip")
    std::map<std::string, Pending> pending_;
    std::map<std::string, std::map<uint32_t, Beat>> beats_;
};

class HubClient {
public:
    ~HubClient();
    HcclResult connect(const std::string &ip, int port, int family, int timeout_ms);
    // All-gather `payload` among the `nmembers` callers that use the same key; out[i] = payload of member i.
    HcclResult rendezvous(const std::string &key, uint32_t nmembers, uint32_t member, const std::string &payload,
                          std::vector<std::string> *out, int timeout_ms);
    HcclResult barrier(const std::string &key, uint32_t nmembers, uint32_t member, int timeout_ms);
    HcclResult heartbeat(const std::string &group, const HeartbeatMsg &msg, HeartbeatSummary *sum, int timeout_ms);
    void bye();
    bool connected() const { return fd_ >= 0; }

private:
    int fd_ = -1;
    std::mutex mu_;
};

}  // namespace hcclb
