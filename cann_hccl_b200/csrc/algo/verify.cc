// Static bounds check of a lowered plan: every step's operand ranges are compared with the sizes of the buffers they
// address before the plan is ever executed.  A schedule bug then shows as HCCL_E_INTERNAL with the offending step at plan
// build time, on the CPU, instead of as a stray access to peer-mapped memory inside a kernel.  Plans are cached, so the
// check runs once per (collective, algorithm, shape).
#include <algorithm>
#include <sstream>
#include "algo/schedule.h"
#include "common/dtype_host.h"

namespace hcclb {
namespace {

struct Bounds {
    uint64_t in = UINT64_MAX, out = UINT64_MAX;  // bytes of the caller's buffers on rank r (UINT64_MAX = not known)
};

uint64_t v_extent(const std::vector<uint64_t> &counts, const std::vector<uint64_t> &displs, int p)
{
    uint64_t m = 0;
    for (int j = 0; j < p && j < (int)counts.size() && j < (int)displs.size(); ++j) m = std::max(m, displs[j] + counts[j]);
    return m;
}

// Sizes that the API contract gives the caller's buffers on rank r, in bytes.
Bounds caller_bounds(const OpDesc &d, int r, int es)
{
    Bounds b;
    const uint64_t n = d.count * (uint64_t)es, p = (uint64_t)d.nranks;
    switch (d.coll) {
        case COLL_ALLREDUCE: case COLL_REDUCE: case COLL_BROADCAST: b.in = b.out = n; break;
        case COLL_ALLGATHER: case COLL_GATHER: b.in = n; b.out = p * n; break;
        case COLL_REDUCE_SCATTER: case COLL_SCATTER: b.in = p * n; b.out = n; break;
        case COLL_ALLTOALL: b.in = b.out = p * n; break;
        case COLL_ALLGATHER_V:
            if ((int)d.counts.size() >= d.nranks && (int)d.displs.size() >= d.nranks) {
                b.in = d.counts[r] * es;
                b.out = v_extent(d.counts, d.displs, d.nranks) * es;
            }
            break;
        case COLL_REDUCE_SCATTER_V:
            if ((int)d.counts.size() >= d.nranks && (int)d.displs.size() >= d.nranks) {
                b.in = v_extent(d.counts, d.displs, d.nranks) * es;
                b.out = d.counts[r] * es;
            }
            break;
        default: break;  // AlltoAllV(C), Send/Recv, Barrier: per-rank layouts, checked through the staging and mailbox bounds only
    }
    return b;
}

}  // namespace

HcclResult verify_plan(const OpDesc &d, const std::vector<int> &local, const Plan &plan, uint64_t stage_half, std::string *why)
{
    const int es = dtype_size(d.dtype), p = d.nranks;
    auto fail = [&](int r, size_t si, const char *what, uint64_t extent, uint64_t bound) {
        std::ostringstream o;
        o << plan.name << ": rank " << r << " step " << si << ": " << what << " reaches byte " << extent << " of " << bound;
        if (why) *why = o.str();
        return HCCL_E_INTERNAL;
    };
    if (plan.steps.size() != local.size()) {
        if (why) *why = plan.name + ": step lists do not match the local ranks";
        return HCCL_E_INTERNAL;
    }
    if (stage_half && plan.stage_bytes > stage_half) return fail(local.empty() ? 0 : local[0], 0, "declared staging need", plan.stage_bytes, stage_half);
    for (size_t li = 0; li < local.size(); ++li) {
        const int r = local[li];
        const Bounds cb = caller_bounds(d, r, es);
        for (size_t si = 0; si < plan.steps[li].size(); ++si) {
            const Step &s = plan.steps[li][si];
            // ---- structure
            auto rank_ok = [&](int16_t q, bool all_allowed) { return q == RANK_SELF || (all_allowed && q == RANK_ALL) || (q >= 0 && q < p); };
            if (s.op > ST_MC_REDUCE) return fail(r, si, "operation code", s.op, ST_MC_REDUCE);
            if (!rank_ok(s.a_rank, true) || !rank_ok(s.b_rank, false) || !rank_ok(s.d_rank, true) || !rank_ok(s.wait_rank, true) || !rank_ok(s.sig_rank, true))
                return fail(r, si, "rank field", 0, (uint64_t)p);
            if (s.chan_n == 0 || (uint32_t)s.chan_lo + s.chan_n > (uint32_t)plan.nchan) return fail(r, si, "channel range", (uint64_t)s.chan_lo + s.chan_n, (uint64_t)plan.nchan);
            if ((s.flags & SF_WAIT_ALLCH) && (uint32_t)s.wait_clo + s.wait_cn > (uint32_t)kMaxChannels)
                return fail(r, si, "producer channel range", (uint64_t)s.wait_clo + s.wait_cn, kMaxChannels);
            if (s.wait_bank >= kFlagBanks || s.sig_bank >= kFlagBanks) return fail(r, si, "flag bank", std::max(s.wait_bank, s.sig_bank), kFlagBanks);
            if (s.op == ST_NOP) continue;
            // ---- operand extents (bytes past the operand's base)
            const uint64_t len = s.count * (uint64_t)es;
            uint64_t a_ext = s.a_off + len, d_ext = s.d_off + len;
            if (s.op == ST_GATHER_ALL) {
                a_ext = d_ext = 0;
                for (int q = 0; q < p; ++q) {
                    uint64_t cnt = s.count;
                    if (s.limit) {
                        uint64_t start = (uint64_t)q * s.count;
                        cnt = start >= s.limit ? 0 : std::min(s.limit - start, s.count);
                    }
                    if (!cnt) continue;
                    a_ext = std::max(a_ext, s.a_off + (uint64_t)q * s.a_stride + cnt * es);
                    d_ext = std::max(d_ext, s.d_off + (uint64_t)q * s.d_stride + cnt * es);
                }
            }
            struct Use { uint8_t buf; uint64_t ext; const char *what; };
            const Use uses[4] = {{s.a_buf, a_ext, "source a"},
                                 {(uint8_t)(s.op == ST_REDUCE2 ? s.b_buf : BUF_NONE), s.b_off + len, "source b"},
                                 {s.d_buf, d_ext, "destination"},
                                 {s.d2_buf, s.d2_off + len, "second destination"}};
            for (const Use &u : uses) {
                if (u.buf == BUF_NONE || len == 0) continue;
                uint64_t bound = UINT64_MAX;
                switch (u.buf) {
                    case BUF_STAGE: bound = plan.stage_bytes; break;
                    case BUF_P2P: bound = (uint64_t)p * d.p2p_slot; break;
                    case BUF_IN: case BUF_ZIN: bound = cb.in; break;
                    case BUF_OUT: case BUF_ZOUT: bound = cb.out; break;
                    default: return fail(r, si, "buffer kind", u.buf, BUF_ZOUT);
                }
                if (bound != UINT64_MAX && u.ext > bound) return fail(r, si, u.what, u.ext, bound);
            }
        }
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
