#include "transport/host_exec.h"
#include <sched.h>
#include <time.h>
#include <cstring>
#include "algo/resolve.h"
#include "common/dtype_host.h"
#include "common/log.h"

namespace hcclb {
namespace {

inline uint64_t now_ns()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

struct Waiter {
    const RankCtx &c;
    uint64_t deadline;
    // Spin until *p >= want.  Returns 0, HCCL_E_TIMEOUT or HCCL_E_SUSPENDING; `seen` gets the last value read.
    int wait_ge(const uint64_t *p, uint64_t want, uint64_t &seen)
    {
        for (uint32_t it = 0;; ++it) {
            seen = __atomic_load_n(p, __ATOMIC_ACQUIRE);
            if (seen >= want) return 0;
            if ((it & 63) == 63) {
                if (c.abort && *c.abort) return *c.abort == 2 ? HCCL_E_REMOTE : HCCL_E_SUSPENDING;
                if (now_ns() > deadline) return HCCL_E_TIMEOUT;
                sched_yield();
            }
        }
    }
};

template <class N>
void reduce2_t(int op, const void *a, const void *b, void *d, void *d2, uint64_t n)
{
    using S = typename N::S;
    const S *pa = (const S *)a, *pb = (const S *)b;
    S *pd = (S *)d, *pd2 = (S *)d2;
    for (uint64_t i = 0; i < n; ++i) {
        S v = N::st(apply_op<typename N::Acc>(op, N::ld(pa[i]), N::ld(pb[i])));
        pd[i] = v;
        if (pd2) pd2[i] = v;
    }
}
template <class N>
void reduce_all_t(int op, const uint8_t *const *src, int p, void *d, void *d2, uint64_t n)
{
    using S = typename N::S;
    S *pd = (S *)d, *pd2 = (S *)d2;
    for (uint64_t i = 0; i < n; ++i) {
        typename N::Acc acc = N::ld(((const S *)src[0])[i]);
        for (int q = 1; q < p; ++q) acc = apply_op<typename N::Acc>(op, acc, N::ld(((const S *)src[q])[i]));
        S v = N::st(acc);
        pd[i] = v;
        if (pd2) pd2[i] = v;
    }
}

void fail(const RankCtx &c, const ExecArgs &a, int code, int step, int peer, int chan, uint64_t want, uint64_t seen)
{
    if (!c.status) return;
    c.status->step = (uint32_t)step;
    c.status->peer = peer;
    c.status->chan = (uint32_t)chan;
    c.status->expected = want;
    c.status->seen = seen;
    c.status->seq = a.seq;
    __atomic_store_n(&c.status->code, (uint32_t)code, __ATOMIC_RELEASE);
}

}  // namespace

HcclResult exec_plan_host(const RankCtx &c, const ExecArgs &a)
{
    const int me = c.rank, p = c.nranks, es = dtype_size(a.dtype);
    Waiter w{c, now_ns() + c.timeout_ns};
    uint64_t half_off = a.track_done ? (a.seq & 1) * c.stage_half : 0;
    uint64_t seen = 0;
    if (a.track_done) {
        if (c.status) __atomic_store_n(&c.status->head, a.seq, __ATOMIC_RELEASE);
        // The staging half of this op was last used by op seq-2: every peer must have left that op.
        if (a.seq >= 2) {
            for (int q = 0; q < p; ++q) {
                if (q == me) continue;
                int rc = w.wait_ge(&c.flags[me][done_index(q)], a.seq - 2, seen);
                if (rc) { fail(c, a, rc, -1, q, 0, a.seq - 2, seen); return (HcclResult)rc; }
            }
        }
    }
    for (int si = 0; si < a.nsteps; ++si) {
        const Step &s = a.steps[si];
        for (int ci = 0; ci < s.chan_n; ++ci) {
            int chan = s.chan_lo + ci;
            if (s.wait_rank != RANK_NONE) {
                uint64_t want = flag_value(a, s, s.wait_val);
                int q0 = s.wait_rank == RANK_ALL ? 0 : s.wait_rank, q1 = s.wait_rank == RANK_ALL ? p : s.wait_rank + 1;
                for (int q = q0; q < q1; ++q) {
                    if (q == me && !(s.flags & SF_INCLUDE_SELF)) continue;
                    int c0 = (s.flags & SF_WAIT_ALLCH) ? s.wait_clo : chan;
                    int c1 = (s.flags & SF_WAIT_ALLCH) ? s.wait_clo + s.wait_cn : chan + 1;
                    for (int cc = c0; cc < c1; ++cc) {
                        int rc = w.wait_ge(&c.flags[me][flag_index(s.wait_bank, q, cc)], want, seen);
                        if (rc) { fail(c, a, rc, si, q, cc, want, seen); return (HcclResult)rc; }
                    }
                }
            }
            uint64_t lo, hi;
            switch (s.op) {
                case ST_COPY: {
                    chan_range(s.count, es, s.chan_n, ci, lo, hi);
                    if (hi > lo) {
                        if (s.d_rank == RANK_ALL) {  // multicast store emulated as a loop over ranks
                            for (int q = 0; q < p; ++q)
                                memmove(resolve_addr(c, a, s.d_buf, q, s.d_off, half_off) + lo * es,
                                        resolve_addr(c, a, s.a_buf, s.a_rank, s.a_off, half_off) + lo * es, (hi - lo) * es);
                        } else {
                            const uint8_t *src = resolve_addr(c, a, s.a_buf, s.a_rank, s.a_off, half_off) + lo * es;
                            memmove(resolve_addr(c, a, s.d_buf, s.d_rank, s.d_off, half_off) + lo * es, src, (hi - lo) * es);
                            if (s.d2_buf != BUF_NONE)
                                memmove(resolve_addr(c, a, s.d2_buf, RANK_SELF, s.d2_off, half_off) + lo * es, src, (hi - lo) * es);
                        }
                    }
                    break;
                }
                case ST_REDUCE2: {
                    chan_range(s.count, es, s.chan_n, ci, lo, hi);
                    if (hi > lo) {
                        const uint8_t *pa = resolve_addr(c, a, s.a_buf, s.a_rank, s.a_off, half_off) + lo * es;
                        const uint8_t *pb = resolve_addr(c, a, s.b_buf, s.b_rank, s.b_off, half_off) + lo * es;
                        uint8_t *pd = resolve_addr(c, a, s.d_buf, s.d_rank, s.d_off, half_off) + lo * es;
                        uint8_t *pd2 = s.d2_buf != BUF_NONE ? resolve_addr(c, a, s.d2_buf, RANK_SELF, s.d2_off, half_off) + lo * es : nullptr;
                        dispatch_reduce_dtype(a.dtype, [&](auto n) { reduce2_t<decltype(n)>(a.redop, pa, pb, pd, pd2, hi - lo); });
                    }
                    break;
                }
                case ST_REDUCE_ALL: case ST_MC_REDUCE: {
                    chan_range(s.count, es, s.chan_n, ci, lo, hi);
                    if (hi > lo) {
                        const uint8_t *src[kMaxRanks];
                        for (int q = 0; q < p; ++q) src[q] = resolve_addr(c, a, s.a_buf, q, s.a_off, half_off) + lo * es;
                        uint8_t *pd2 = s.d2_buf != BUF_NONE ? resolve_addr(c, a, s.d2_buf, RANK_SELF, s.d2_off, half_off) + lo * es : nullptr;
                        if (s.d_rank == RANK_ALL) {  // reduce then multicast store
                            uint8_t *first = resolve_addr(c, a, s.d_buf, 0, s.d_off, half_off) + lo * es;
                            dispatch_reduce_dtype(a.dtype, [&](auto n) { reduce_all_t<decltype(n)>(a.redop, src, p, first, pd2, hi - lo); });
                            for (int q = 1; q < p; ++q)
                                memcpy(resolve_addr(c, a, s.d_buf, q, s.d_off, half_off) + lo * es, first, (hi - lo) * es);
                        } else {
                            uint8_t *pd = resolve_addr(c, a, s.d_buf, s.d_rank, s.d_off, half_off) + lo * es;
                            dispatch_reduce_dtype(a.dtype, [&](auto n) { reduce_all_t<decltype(n)>(a.redop, src, p, pd, pd2, hi - lo); });
                        }
                    }
                    break;
                }
                case ST_GATHER_ALL: {
                    for (int i = 0; i < p; ++i) {
                        int q = (me + i) % p;
                        if (q == me && (s.flags & SF_SKIP_SELF)) continue;
                        uint64_t cnt = s.count;
                        if (s.limit) {
                            uint64_t start = (uint64_t)q * s.count;
                            cnt = start >= s.limit ? 0 : (s.limit - start < s.count ? s.limit - start : s.count);
                        }
                        chan_range(cnt, es, s.chan_n, ci, lo, hi);
                        if (hi <= lo) continue;
                        int src_rank = s.a_rank == RANK_ALL ? q : RANK_SELF;
                        memmove(resolve_addr(c, a, s.d_buf, RANK_SELF, s.d_off + (uint64_t)q * s.d_stride, half_off) + lo * es,
                                resolve_addr(c, a, s.a_buf, src_rank, s.a_off + (uint64_t)q * s.a_stride, half_off) + lo * es,
                                (hi - lo) * es);
                    }
                    break;
                }
                default: break;
            }
            if (s.sig_rank != RANK_NONE) {
                uint64_t val = flag_value(a, s, s.sig_val);
                int q0 = s.sig_rank == RANK_ALL ? 0 : s.sig_rank, q1 = s.sig_rank == RANK_ALL ? p : s.sig_rank + 1;
                for (int q = q0; q < q1; ++q) {
                    if (q == me && !(s.flags & SF_INCLUDE_SELF)) continue;
                    __atomic_store_n(&c.flags[q][flag_index(s.sig_bank, me, chan)], val, __ATOMIC_RELEASE);
                }
            }
        }
    }
    if (a.track_done) {
        for (int q = 0; q < p; ++q)
            if (q != me) __atomic_store_n(&c.flags[q][done_index(me)], a.seq, __ATOMIC_RELEASE);
        if (c.status) __atomic_store_n(&c.status->tail, a.seq, __ATOMIC_RELEASE);
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
