// Static race detection for a lowered plan.
//
// On the GPU every channel of every rank is a CTA of its own, and nothing orders two CTAs except the flag waits of the
// plan.  The CPU executor runs the channels of a rank one after the other, so a missing dependency between two channels of
// one rank, or between channels of different ranks that happen to be scheduled in a lucky order, never shows there.  This
// check needs neither: it builds the happens-before relation of the plan (program order of every (rank, channel) pair plus
// one edge from the step that sends a flag value to every step that waits for it) and then demands that any two accesses
// to overlapping bytes of the same buffer, one of them a write, are ordered by it.  It also reports waits that no step
// ever satisfies and cycles of waits (both would end in a timeout).
//
// The reference has no such tool; its templates rely on review and on the stream / notify order of the runtime
// (algorithm/base/alg_template/**).  In-place calls are modelled by folding the caller's two buffers into one, with the
// offset that the collective's in-place form prescribes (algorithm/impl/coll_alg_utils.cc:253-307).
#include <algorithm>
#include <map>
#include <sstream>
#include <tuple>
#include "algo/schedule.h"
#include "common/dtype_host.h"

namespace hcclb {
namespace {

struct Access {
    int node;
    uint64_t lo, hi;  // bytes
    bool write;
};

struct Node {
    int rank, step, chan;
};

// Buffer instance: (owning rank, kind).  In place, the receive buffer of a rank is folded onto its send buffer.
using BufKey = std::pair<int, int>;

}  // namespace

HcclResult race_check_plan(const OpDesc &d, const Plan &plan, bool in_place, std::string *why)
{
    const int p = d.nranks, es = dtype_size(d.dtype);
    auto fail = [&](const std::string &msg) {
        if (why) *why = plan.name + ": " + msg;
        return HCCL_E_INTERNAL;
    };
    if ((int)plan.steps.size() != p) return fail("the race check needs the step lists of all ranks");

    // ---- nodes: one per (rank, step, channel that executes the step), in program order per (rank, channel)
    std::vector<Node> nodes;
    std::vector<std::vector<std::vector<int>>> node_of(p);  // [rank][step][channel - chan_lo]
    for (int r = 0; r < p; ++r) {
        node_of[r].resize(plan.steps[r].size());
        for (size_t si = 0; si < plan.steps[r].size(); ++si) {
            const Step &s = plan.steps[r][si];
            if (s.flags & SF_ABS_VALS) return fail("plans with absolute flag values (Send / Recv) are outside this check");
            for (int ci = 0; ci < s.chan_n; ++ci) {
                node_of[r][si].push_back((int)nodes.size());
                nodes.push_back({r, (int)si, s.chan_lo + ci});
            }
        }
    }
    const int N = (int)nodes.size();
    std::vector<std::vector<int>> preds(N);
    auto node_at = [&](int r, int si, int chan) {
        const Step &s = plan.steps[r][si];
        return (chan >= s.chan_lo && chan < s.chan_lo + s.chan_n) ? node_of[r][si][chan - s.chan_lo] : -1;
    };
    for (int r = 0; r < p; ++r) {
        std::map<int, int> last;  // channel -> newest node
        for (size_t si = 0; si < plan.steps[r].size(); ++si) {
            const Step &s = plan.steps[r][si];
            for (int ci = 0; ci < s.chan_n; ++ci) {
                const int chan = s.chan_lo + ci, n = node_of[r][si][ci];
                auto it = last.find(chan);
                if (it != last.end()) preds[n].push_back(it->second);
                last[chan] = n;
            }
        }
    }
    // ---- flag edges: the first step of (producer rank, producer channel) whose signal reaches the waiting rank on the same
    // bank with a value of at least the awaited one (values only grow along a step list)
    for (int n = 0; n < N; ++n) {
        const Node &nd = nodes[n];
        const Step &s = plan.steps[nd.rank][nd.step];
        if (s.wait_rank == RANK_NONE) continue;
        const int q0 = s.wait_rank == RANK_ALL ? 0 : s.wait_rank, q1 = s.wait_rank == RANK_ALL ? p : s.wait_rank + 1;
        for (int q = q0; q < q1; ++q) {
            if (q == nd.rank && !(s.flags & SF_INCLUDE_SELF)) continue;
            const int c0 = (s.flags & SF_WAIT_ALLCH) ? s.wait_clo : nd.chan;
            const int c1 = (s.flags & SF_WAIT_ALLCH) ? s.wait_clo + s.wait_cn : nd.chan + 1;
            for (int cc = c0; cc < c1; ++cc) {
                int found = -1;
                for (size_t sj = 0; sj < plan.steps[q].size() && found < 0; ++sj) {
                    const Step &t = plan.steps[q][sj];
                    if (t.sig_rank == RANK_NONE || t.sig_bank != s.wait_bank || t.sig_val < s.wait_val) continue;
                    const bool reaches = t.sig_rank == RANK_ALL ? (q != nd.rank || (t.flags & SF_INCLUDE_SELF))
                                                                : (t.sig_rank == nd.rank && (q != nd.rank || (t.flags & SF_INCLUDE_SELF)));
                    if (!reaches) continue;
                    found = node_at(q, (int)sj, cc);
                }
                if (found < 0) {
                    std::ostringstream o;
                    o << "rank " << nd.rank << " step " << nd.step << " channel " << nd.chan << " waits for value " << s.wait_val << " from rank " << q
                      << " channel " << cc << ", which no step sends";
                    return fail(o.str());
                }
                preds[n].push_back(found);
            }
        }
    }
    // ---- ancestors by a topological sweep (a cycle is a deadlock)
    const int W = (N + 63) / 64;
    std::vector<uint64_t> anc((size_t)N * W, 0);
    std::vector<int> indeg(N, 0), order;
    std::vector<std::vector<int>> succs(N);
    for (int n = 0; n < N; ++n)
        for (int q : preds[n]) { succs[q].push_back(n); ++indeg[n]; }
    for (int n = 0; n < N; ++n)
        if (!indeg[n]) order.push_back(n);
    for (size_t i = 0; i < order.size(); ++i) {
        const int n = order[i];
        for (int m : succs[n]) {
            uint64_t *am = &anc[(size_t)m * W];
            const uint64_t *an = &anc[(size_t)n * W];
            for (int w = 0; w < W; ++w) am[w] |= an[w];
            am[n / 64] |= 1ull << (n % 64);
            if (--indeg[m] == 0) order.push_back(m);
        }
    }
    if ((int)order.size() != N) return fail("the waits of the plan form a cycle (deadlock)");
    auto before = [&](int a, int b) { return (anc[(size_t)b * W + a / 64] >> (a % 64)) & 1ull; };

    // ---- accesses
    const uint64_t n_bytes = d.count * (uint64_t)es;
    auto key_of = [&](int owner, uint8_t buf, uint64_t &shift) {
        shift = 0;
        int kind = buf;
        if (kind == BUF_ZIN) kind = BUF_IN;
        if (kind == BUF_ZOUT) kind = BUF_OUT;
        if (in_place) {
            // fold the receive buffer onto the send buffer (or the other way round) as the in-place form of the collective puts them
            switch (d.coll) {
                case COLL_ALLREDUCE: case COLL_REDUCE: case COLL_BROADCAST:
                    if (kind == BUF_OUT) kind = BUF_IN;
                    break;
                case COLL_ALLGATHER: case COLL_GATHER:  // the send buffer is block `owner` of the receive buffer
                    if (kind == BUF_IN) { kind = BUF_OUT; shift = (uint64_t)owner * n_bytes; }
                    break;
                case COLL_REDUCE_SCATTER: case COLL_SCATTER:  // the receive buffer is block `owner` of the send buffer
                    if (kind == BUF_OUT) { kind = BUF_IN; shift = (uint64_t)owner * n_bytes; }
                    break;
                default: break;
            }
        }
        return BufKey(owner, kind);
    };
    std::map<BufKey, std::vector<Access>> acc;
    auto add = [&](int n, int owner, uint8_t buf, uint64_t off, uint64_t lo_e, uint64_t hi_e, bool write) {
        if (buf == BUF_NONE || hi_e <= lo_e) return;
        uint64_t shift;
        BufKey k = key_of(owner, buf, shift);
        acc[k].push_back({n, shift + off + lo_e * es, shift + off + hi_e * es, write});
    };
    for (int n = 0; n < N; ++n) {
        const Node &nd = nodes[n];
        const Step &s = plan.steps[nd.rank][nd.step];
        const int me = nd.rank, ci = nd.chan - s.chan_lo;
        auto owner = [&](int16_t rk) { return rk == RANK_SELF ? me : (int)rk; };
        uint64_t lo, hi;
        switch (s.op) {
            case ST_COPY: case ST_REDUCE2: {
                chan_range(s.count, es, s.chan_n, ci, lo, hi);
                add(n, owner(s.a_rank), s.a_buf, s.a_off, lo, hi, false);
                if (s.op == ST_REDUCE2) add(n, owner(s.b_rank), s.b_buf, s.b_off, lo, hi, false);
                if (s.d_rank == RANK_ALL)
                    for (int q = 0; q < p; ++q) add(n, q, s.d_buf, s.d_off, lo, hi, true);
                else add(n, owner(s.d_rank), s.d_buf, s.d_off, lo, hi, true);
                add(n, me, s.d2_buf, s.d2_off, lo, hi, true);
                break;
            }
            case ST_REDUCE_ALL: case ST_MC_REDUCE: {
                chan_range(s.count, es, s.chan_n, ci, lo, hi);
                for (int q = 0; q < p; ++q) add(n, q, s.a_buf, s.a_off, lo, hi, false);
                if (s.d_rank == RANK_ALL)
                    for (int q = 0; q < p; ++q) add(n, q, s.d_buf, s.d_off, lo, hi, true);
                else add(n, owner(s.d_rank), s.d_buf, s.d_off, lo, hi, true);
                add(n, me, s.d2_buf, s.d2_off, lo, hi, true);
                break;
            }
            case ST_GATHER_ALL: {
                for (int q = 0; q < p; ++q) {
                    if (q == me && (s.flags & SF_SKIP_SELF)) continue;
                    uint64_t cnt = s.count;
                    if (s.limit) {
                        const uint64_t start = (uint64_t)q * s.count;
                        cnt = start >= s.limit ? 0 : (s.limit - start < s.count ? s.limit - start : s.count);
                    }
                    chan_range(cnt, es, s.chan_n, ci, lo, hi);
                    add(n, s.a_rank == RANK_ALL ? q : me, s.a_buf, s.a_off + (uint64_t)q * s.a_stride, lo, hi, false);
                    add(n, me, s.d_buf, s.d_off + (uint64_t)q * s.d_stride, lo, hi, true);
                }
                break;
            }
            default: break;
        }
    }
    // ---- conflicting accesses must be ordered
    for (auto &kv : acc) {
        std::vector<Access> &v = kv.second;
        std::sort(v.begin(), v.end(), [](const Access &x, const Access &y) { return x.lo < y.lo; });
        for (size_t i = 0; i < v.size(); ++i) {
            for (size_t j = i + 1; j < v.size() && v[j].lo < v[i].hi; ++j) {
                if (!(v[i].write || v[j].write) || v[i].node == v[j].node) continue;
                const int a = v[i].node, b = v[j].node;
                if (before(a, b) || before(b, a)) continue;
                const Node &na = nodes[a], &nb = nodes[b];
                static const char *kinds[] = {"send buffer", "receive buffer", "staging", "mailbox", "send buffer", "receive buffer", "?", "?"};
                std::ostringstream o;
                o << "unordered " << (v[i].write ? "write" : "read") << " / " << (v[j].write ? "write" : "read") << " on the " << kinds[kv.first.second & 7]
                  << " of rank " << kv.first.first << ", bytes [" << std::max(v[i].lo, v[j].lo) << ", " << std::min(v[i].hi, v[j].hi) << "): rank "
                  << na.rank << " step " << na.step << " channel " << na.chan << " and rank " << nb.rank << " step " << nb.step << " channel " << nb.chan;
                return fail(o.str());
            }
        }
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
