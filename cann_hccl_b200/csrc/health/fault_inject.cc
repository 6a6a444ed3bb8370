#include "health/fault_inject.h"
#include <unistd.h>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>
#include "common/log.h"
namespace hcclb {
namespace fault {
namespace {
struct Rule { std::string kind; long rank = -1, op = -1, ms = 0, after = 0, attempts = 0; };
std::vector<Rule> g_rules;
std::mutex g_mu;
bool g_loaded = false;
std::atomic<long> g_beats{0};
long field(const std::string &s, const char *name, long dflt)
{
    size_t p = s.find(std::string(name) + "=");
    return p == std::string::npos ? dflt : strtol(s.c_str() + p + strlen(name) + 1, nullptr, 10);
}
void load_locked()
{
    g_rules.clear();
    g_loaded = true;
    const char *e = getenv("HCCL_FAULT_INJECT");
    if (!e) return;
    std::string all = e;
    size_t pos = 0;
    while (pos <= all.size()) {
        size_t end = all.find(';', pos);
        std::string item = all.substr(pos, end == std::string::npos ? std::string::npos : end - pos);
        if (!item.empty()) {
            Rule r;
            size_t c = item.find(':');
            r.kind = item.substr(0, c);
            std::string args = c == std::string::npos ? "" : item.substr(c + 1);
            r.rank = field(args, "rank", -1);
            r.op = field(args, "op", -1);
            r.ms = field(args, "ms", 0);
            r.after = field(args, "after", 0);
            r.attempts = field(args, "attempts", 0);
            g_rules.push_back(r);
        }
        if (end == std::string::npos) break;
        pos = end + 1;
    }
}
}  // namespace
void reload()
{
    std::lock_guard<std::mutex> lk(g_mu);
    load_locked();
}
void before_op(int rank, uint64_t op_index)
{
    std::vector<Rule> rules;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_loaded) load_locked();
        rules = g_rules;
    }
    for (auto &r : rules) {
        if (r.rank != rank || r.op != (long)op_index) continue;
        if (r.kind == "stall_rank") {
            HLOG_WARN("fault injection: rank %d stalls %ld ms before op %llu", rank, r.ms, (unsigned long long)op_index);
            usleep((useconds_t)r.ms * 1000);
        } else if (r.kind == "exit_rank") {
            HLOG_WARN("fault injection: rank %d exits before op %llu", rank, (unsigned long long)op_index);
            _exit(17);
        }
    }
}
void before_attempt(int rank, uint64_t op_index, int attempt)
{
    std::vector<Rule> rules;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_loaded) load_locked();
        rules = g_rules;
    }
    for (auto &r : rules)
        if (r.kind == "stall_rank" && r.rank == rank && r.op == (long)op_index && attempt <= r.attempts) {
            HLOG_WARN("fault injection: rank %d stalls %ld ms before retry %d of op %llu", rank, r.ms, attempt, (unsigned long long)op_index);
            usleep((useconds_t)r.ms * 1000);
        }
}
bool drop_heartbeat(int rank)
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_loaded) load_locked();
    for (auto &r : g_rules)
        if (r.kind == "drop_heartbeat" && r.rank == rank) return g_beats.fetch_add(1) >= r.after;
    return false;
}
}  // namespace fault
}  // namespace hcclb
