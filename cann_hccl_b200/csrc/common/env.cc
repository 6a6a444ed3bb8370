#include "common/env.h"
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include "common/log.h"

extern char **environ;
namespace hcclb {

static std::string lower(std::string s)
{
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)tolower(c); });
    return s;
}
static bool parse_int(const std::string &s, long &out)
{
    if (s.empty()) return false;
    char *end = nullptr;
    out = strtol(s.c_str(), &end, 10);
    return end && *end == 0;
}
static void fail(EnvConfig &c, const std::string &msg)
{
    if (c.valid) c.error = msg;
    c.valid = false;
}

EnvConfig parse_env(const std::map<std::string, std::string> &v)
{
    EnvConfig c;
    auto get = [&](const char *k) -> const std::string * {
        auto it = v.find(k);
        return it == v.end() ? nullptr : &it->second;
    };
    long n;
    if (auto s = get("HCCL_ALGO")) {
        // Accepted: "ring" (all ops), "allreduce=ring;allgather=mesh", and the reference's
        // "level0:NA;level1:ring" form (only the last level named matters on one NVSwitch domain).
        std::string str = lower(*s);
        size_t pos = 0;
        while (pos <= str.size()) {
            size_t e = str.find(';', pos);
            std::string item = str.substr(pos, e == std::string::npos ? std::string::npos : e - pos);
            if (!item.empty()) {
                size_t eq = item.find_first_of("=:");
                std::string key = eq == std::string::npos ? "*" : item.substr(0, eq);
                std::string val = eq == std::string::npos ? item : item.substr(eq + 1);
                if (key.rfind("level", 0) == 0) key = "*";
                if (val != "na" && !val.empty()) c.algo[key] = val;
            }
            if (e == std::string::npos) break;
            pos = e + 1;
        }
    }
    if (auto s = get("HCCL_BUFFSIZE")) {
        if (parse_int(*s, n) && n >= 1 && n <= 65536) { c.buffsize_mb = (uint32_t)n; c.buffsize_set = true; }
        else fail(c, "HCCL_BUFFSIZE must be an integer number of MB >= 1");
    }
    if (auto s = get("HCCL_DETERMINISTIC")) {
        std::string l = lower(*s);
        if (l == "true" || l == "1") c.deterministic = 1;
        else if (l == "false" || l == "0") c.deterministic = 0;
        else fail(c, "HCCL_DETERMINISTIC must be true/false");
    }
    if (auto s = get("HCCL_OP_EXPANSION_MODE")) {
        std::string l = lower(*s);
        if (l == "host") c.expansion_mode = 1;
        else if (l == "ai_cpu" || l == "aicpu") c.expansion_mode = 2;
        else if (l == "aiv" || l == "device") c.expansion_mode = 3;
        else if (l == "auto" || l == "0") c.expansion_mode = 0;
        else fail(c, "HCCL_OP_EXPANSION_MODE must be HOST, AI_CPU, AIV or AUTO");
    }
    if (auto s = get("HCCL_CONNECT_TIMEOUT")) {
        if (parse_int(*s, n) && n >= 1 && n <= 7200) c.connect_timeout_s = (int)n;
        else fail(c, "HCCL_CONNECT_TIMEOUT must be in [1,7200] seconds");
    }
    if (auto s = get("HCCL_EXEC_TIMEOUT")) {
        if (parse_int(*s, n) && n >= 0 && n <= 2147483647) c.exec_timeout_s = (int)n;
        else fail(c, "HCCL_EXEC_TIMEOUT must be a non-negative number of seconds");
    }
    if (auto s = get("HCCL_EXEC_TIMEOUT_MS")) c.exec_timeout_ms = atof(s->c_str());
    if (auto s = get("HCCL_IF_BASE_PORT")) {
        if (parse_int(*s, n) && n >= 1024 && n <= 65520) c.if_base_port = (int)n;
        else fail(c, "HCCL_IF_BASE_PORT must be in [1024,65520]");
    }
    if (auto s = get("HCCL_IF_IP")) c.if_ip = *s;
    if (auto s = get("HCCL_SOCKET_FAMILY")) {
        std::string l = lower(*s);
        if (l == "af_inet") c.socket_family = 4;
        else if (l == "af_inet6") c.socket_family = 6;
        else fail(c, "HCCL_SOCKET_FAMILY must be AF_INET or AF_INET6");
    }
    if (auto s = get("HCCL_OP_RETRY_ENABLE")) {
        std::string l = lower(*s);
        c.retry_enable = l.find(":1") != std::string::npos || l == "1" || l == "true";
    }
    if (auto s = get("HCCL_OP_RETRY_PARAMS")) {
        // "MaxCnt:3,HoldTime:5000,IntervalTime:1000"
        std::string l = lower(*s);
        auto field = [&](const char *name, int &dst, long lo, long hi) {
            size_t p = l.find(name);
            if (p == std::string::npos) return;
            p = l.find(':', p);
            if (p == std::string::npos) return;
            long val = strtol(l.c_str() + p + 1, nullptr, 10);
            if (val < lo || val > hi) fail(c, std::string("HCCL_OP_RETRY_PARAMS ") + name + " out of range");
            else dst = (int)val;
        };
        field("maxcnt", c.retry_max, 1, 10);
        field("holdtime", c.retry_hold_ms, 0, 60000);
        field("intervaltime", c.retry_interval_ms, 0, 60000);
    }
    if (auto s = get("HCCL_ENTRY_LOG_ENABLE")) c.entry_log = (*s == "1");
    if (auto s = get("HCCL_OP_COUNTER")) c.op_counter = (*s != "0");
    if (auto s = get("HCCL_NVLS_ENABLE")) {
        if (parse_int(*s, n) && (n == 0 || n == 1)) c.nvls_enable = (int)n;
        else fail(c, "HCCL_NVLS_ENABLE must be 0 or 1");
    }
    if (auto s = get("HCCL_TRANSPORT")) {
        c.transport = lower(*s);
        if (c.transport != "host" && c.transport != "p2p" && !c.transport.empty())
            fail(c, "HCCL_TRANSPORT must be host or p2p");
    }
    if (auto s = get("HCCL_FAULT_INJECT")) c.fault_inject = *s;
    if (auto s = get("HCCL_RDMA_TC")) {
        if (parse_int(*s, n) && n >= 0 && n <= 255 && n % 4 == 0) c.rdma_tc = (int)n;
        else fail(c, "HCCL_RDMA_TC must be in [0,255] and a multiple of 4");
    }
    if (auto s = get("HCCL_RDMA_SL")) {
        if (parse_int(*s, n) && n >= 0 && n <= 7) c.rdma_sl = (int)n;
        else fail(c, "HCCL_RDMA_SL must be in [0,7]");
    }
    if (auto s = get("HCCL_HOST_SOCKET_PORT_RANGE")) {
        int lo = 0, hi = 0;
        if (sscanf(s->c_str(), "%d-%d", &lo, &hi) == 2 && lo >= 1 && hi <= 65535 && lo <= hi) {
            c.port_range_lo = lo; c.port_range_hi = hi;
        } else if (lower(*s) != "auto") fail(c, "HCCL_HOST_SOCKET_PORT_RANGE must be lo-hi or auto");
    }
    if (auto s = get("HCCL_HEARTBEAT_INTERVAL_MS")) { if (parse_int(*s, n) && n >= 1) c.heartbeat_ms = (int)n; }
    if (auto s = get("HCCL_HEARTBEAT_LOST_MS")) { if (parse_int(*s, n) && n >= 1) c.heartbeat_lost_ms = (int)n; }
    if (auto s = get("HCCL_STUCK_DETECT_TIME")) { if (parse_int(*s, n) && n >= 1) c.stuck_ms = (int)n * 1000; }
    if (auto s = get("HCCL_STUCK_DETECT_MS")) { if (parse_int(*s, n) && n >= 1) c.stuck_ms = (int)n; }
    if (auto s = get("HCCL_ALLTOALLV_CHECK")) { if (parse_int(*s, n) && (n == 0 || n == 1)) c.a2av_check = (int)n; else fail(c, "HCCL_ALLTOALLV_CHECK must be 0 or 1"); }
    if (auto s = get("HCCL_CALIBRATE")) c.calibrate = !(*s == "0" || lower(*s) == "false");
    if (auto s = get("HCCL_CALIBRATE_MAX_MB")) { if (parse_int(*s, n) && n >= 1 && n <= 1024) c.calibrate_max_mb = (int)n; }
    if (auto s = get("HCCL_CHANNELS")) { if (parse_int(*s, n) && n >= 0 && n <= 128) c.channels = (int)n; }
    if (auto s = get("HCCL_PIPE_CHUNK_KB")) { if (parse_int(*s, n) && n >= 16) c.pipe_chunk_bytes = (uint64_t)n << 10; }
    if (auto s = get("HCCL_PIPE_SLOTS")) { if (parse_int(*s, n) && n >= 1 && n <= 16) c.pipe_slots = (int)n; }
    if (auto s = get("HCCL_PIPE_CTAS")) {
        int a = 0, b = 0, d = 0;
        if (sscanf(s->c_str(), "%d,%d,%d", &a, &b, &d) >= 2 && a >= 1 && b >= 1 && d >= 0 && a + b + d <= 128) { c.pipe_ctas[0] = a; c.pipe_ctas[1] = b; c.pipe_ctas[2] = d > 0 ? d : 1; }
        else fail(c, "HCCL_PIPE_CTAS must be a,b[,c] with a + b + c <= 128");
    }
    if (auto s = get("HCCL_PIPE_GROUPS")) {
        int a = 0, b = 0, d = 0;
        if (sscanf(s->c_str(), "%d,%d,%d", &a, &b, &d) >= 2 && a >= 1 && b >= 1 && d >= 0 && a <= 16 && b <= 16 && d <= 16) { c.pipe_groups[0] = a; c.pipe_groups[1] = b; c.pipe_groups[2] = d > 0 ? d : 1; }
        else fail(c, "HCCL_PIPE_GROUPS must be a,b[,c] with values in [1,16]");
    }
    if (auto s = get("HCCL_PLAN_RACE_CHECK")) c.plan_race_check = *s == "1" || lower(*s) == "true";
    if (auto s = get("HCCL_TP_GEMM_PAIR")) c.tp_gemm_pair = !(*s == "0" || lower(*s) == "false");
    if (auto s = get("HCCL_NCCL_LIB")) c.ncc_lib = *s;
    if (auto s = get("HCCL_WHITELIST_DISABLE")) c.whitelist_enable = *s == "0";
    if (auto s = get("HCCL_WHITELIST_FILE")) c.whitelist_file = *s;
    if (c.whitelist_enable && c.whitelist_file.empty()) fail(c, "HCCL_WHITELIST_DISABLE=0 needs HCCL_WHITELIST_FILE");
    if (auto s = get("HCCL_NVTX")) c.nvtx = *s == "1" || lower(*s) == "true";
    if (auto s = get("HCCL_OVERFLOW_CHECK")) c.overflow_check = *s == "1" || lower(*s) == "true";
    if (auto s = get("HCCL_STATS_DUMP")) c.stats_dump = *s;
    return c;
}

const EnvConfig &env_config(bool force)
{
    static EnvConfig cfg;
    static bool init = false;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    if (!init || force) {
        std::map<std::string, std::string> vars;
        for (char **e = environ; e && *e; ++e) {
            if (strncmp(*e, "HCCL_", 5) != 0) continue;
            const char *eq = strchr(*e, '=');
            if (!eq) continue;
            vars[std::string(*e, eq - *e)] = std::string(eq + 1);
        }
        cfg = parse_env(vars);
        if (!cfg.valid) HLOG_ERROR("environment configuration error: %s", cfg.error.c_str());
        init = true;
    }
    return cfg;
}
}  // namespace hcclb
