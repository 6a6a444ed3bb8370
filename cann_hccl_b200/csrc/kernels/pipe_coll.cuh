// Pipelined large-message kernel for sm_100a: see pipe_coll.h for the role it plays.  One kernel per (element type,
// reduction operator), instantiated next to the plan executor of the same type.
//
// Protocol.  The op's half of the staging buffer is a ring of `nslots` slots; chunk c lives in slot c % nslots on every
// rank.  The CTAs of a rank form up to three stages.  Every CTA of a stage works on its share of every chunk; when it is
// done with a chunk it adds one to that slot's arrival counter (gpu scope), and the CTA that arrives last publishes the
// stage's progress, (seq << kSeqShift) + c + 1, with ONE st.release.sys per destination rank (its own page included, for
// the next stage of the same rank).  A stage starts chunk c when the progress words it depends on have reached c + 1,
// and a stage writes into a slot again only after every reader of the chunk that lived there has published its
// progress, so the ring needs no other hand-shake.  Every dependency points to an earlier stage of the same chunk or
// to an earlier chunk, so the stages cannot wait on one another in a cycle.  All waits are bounded (wait_flag_ge); a
// CTA that gives up records the status block and every other CTA of the rank leaves at its next wait.
#pragma once
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.h"

namespace hcclb {

// d[q] = reduction over the p sources in rank order, for every destination q (two-shot AllReduce over peer mappings).
template <class T, int OP>
__device__ __forceinline__ void reduce_to_all_range(const uint8_t *const *src, uint8_t *const *dst, int p, uint64_t n)
{
    using N = DNum<T>;
    using Acc = typename N::Acc;
    const int tid = threadIdx.x, nt = blockDim.x;
    constexpr int E = 16 / sizeof(T);
    bool al = true;
    for (int q = 0; q < p; ++q) al = al && aligned16(src[q]) && aligned16(dst[q]);
    uint64_t done = 0;
    if (al && p <= 8) {
        // one vector from each of up to eight ranks in flight per thread, then one store per rank
        const uint64_t nvec = n / E;
        for (uint64_t i = tid; i < nvec; i += nt) {
            uint4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (q < p) v[q] = ld_stream((const uint4 *)src[q] + i);
            Acc acc[E];
            Pack16<T> t;
            t.u = v[0];
#pragma unroll
            for (int k = 0; k < E; ++k) acc[k] = N::up(t.e[k]);
#pragma unroll
            for (int q = 1; q < 8; ++q)
                if (q < p) {
                    Pack16<T> y;
                    y.u = v[q];
#pragma unroll
                    for (int k = 0; k < E; ++k) acc[k] = red_op<OP>(acc[k], N::up(y.e[k]));
                }
            Pack16<T> z;
#pragma unroll
            for (int k = 0; k < E; ++k) z.e[k] = N::down(acc[k]);
#pragma unroll
            for (int q = 0; q < 8; ++q)
                if (q < p) ((uint4 *)dst[q])[i] = z.u;
        }
        done = nvec * E;
    }
    for (uint64_t i = done + tid; i < n; i += nt) {
        Acc acc = N::up(((const T *)src[0])[i]);
        for (int q = 1; q < p; ++q) acc = red_op<OP>(acc, N::up(((const T *)src[q])[i]));
        T v = N::down(acc);
        for (int q = 0; q < p; ++q) ((T *)dst[q])[i] = v;
    }
}

// The transfer loops are kept out of line: each gets its own register allocation (they hold up to 16 vectors per thread),
// and the stage loop around them stays small.
static __device__ __noinline__ void pipe_copy(const uint8_t *a, uint8_t *d, uint8_t *d2, uint64_t bytes, int es) { copy_range(a, d, d2, bytes, es); }

// d = a with sixteen vectors in flight per thread: for peer loads, whose round trip over NVLink takes microseconds
static __device__ __noinline__ void pipe_copy_deep(const uint8_t *a, uint8_t *d, uint64_t bytes, int es)
{
    if (!(aligned16(a) && aligned16(d))) { copy_range(a, d, nullptr, bytes, es); return; }
    const int tid = threadIdx.x, nt = blockDim.x;
    const uint64_t nvec = bytes >> 4;
    constexpr int U = 16;
    for (uint64_t i = tid; i < nvec; i += (uint64_t)U * nt) {
        uint4 v[U];
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (i + (uint64_t)k * nt < nvec) v[k] = ld_stream((const uint4 *)a + i + (uint64_t)k * nt);
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (i + (uint64_t)k * nt < nvec) ((uint4 *)d)[i + (uint64_t)k * nt] = v[k];
    }
    for (uint64_t b = (nvec << 4) + tid; b < bytes; b += nt) d[b] = a[b];
}

// np independent copies (piece k: bytes[k] from src[k] to dst[k]); two vectors of each of eight pieces in flight per thread
static __device__ __noinline__ void pipe_copy_pieces(const uint8_t *const *src, uint8_t *const *dst, const uint64_t *bytes, int np, int es)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    bool fast = true;
    uint64_t mx = 0;
    for (int k = 0; k < np; ++k) {
        fast = fast && aligned16(src[k]) && aligned16(dst[k]) && (bytes[k] & 15) == 0;
        mx = bytes[k] > mx ? bytes[k] : mx;
    }
    if (!fast) {
        for (int k = 0; k < np; ++k)
            if (bytes[k]) copy_range(src[k], dst[k], nullptr, bytes[k], es);
        return;
    }
    const uint64_t nvec = mx >> 4;
    for (int k0 = 0; k0 < np; k0 += 8) {
        for (uint64_t i = tid; i < nvec; i += 2ull * nt) {
            uint4 v[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k0 + k < np && ((i + (uint64_t)u * nt) << 4) < bytes[k0 + k]) v[u][k] = ld_stream((const uint4 *)src[k0 + k] + i + (uint64_t)u * nt);
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k0 + k < np && ((i + (uint64_t)u * nt) << 4) < bytes[k0 + k]) ((uint4 *)dst[k0 + k])[i + (uint64_t)u * nt] = v[u][k];
        }
    }
}

// dst[q] = a for nd destinations: one load, nd stores
static __device__ __noinline__ void pipe_copy_bcast(const uint8_t *a, uint8_t *const *dst, int nd, uint64_t bytes, int es)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    bool fast = aligned16(a);
    for (int q = 0; q < nd; ++q) fast = fast && aligned16(dst[q]);
    if (!fast) {
        for (int q = 0; q < nd; ++q) copy_range(a, dst[q], nullptr, bytes, es);
        return;
    }
    const uint64_t nvec = bytes >> 4;
    constexpr int U = 8;
    for (uint64_t i = tid; i < nvec; i += (uint64_t)U * nt) {
        uint4 v[U];
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (i + (uint64_t)k * nt < nvec) v[k] = ld_stream((const uint4 *)a + i + (uint64_t)k * nt);
        for (int q = 0; q < nd; ++q) {
#pragma unroll
            for (int k = 0; k < U; ++k)
                if (i + (uint64_t)k * nt < nvec) ((uint4 *)dst[q])[i + (uint64_t)k * nt] = v[k];
        }
    }
    for (uint64_t b = (nvec << 4) + tid; b < bytes; b += nt) {
        const uint8_t x = a[b];
        for (int q = 0; q < nd; ++q) dst[q][b] = x;
    }
}

__device__ __forceinline__ uint4 ld_any16(const uint8_t *a)
{
    Pack16<uint8_t> t;
    if ((((uintptr_t)a) & 3) == 0) {
        Pack16<uint32_t> w;
#pragma unroll
        for (int k = 0; k < 4; ++k) w.e[k] = ((const uint32_t *)a)[k];
        return w.u;
    }
#pragma unroll
    for (int k = 0; k < 16; ++k) t.e[k] = a[k];
    return t.u;
}
__device__ __forceinline__ void st_any16(uint8_t *d, uint4 v)
{
    if ((((uintptr_t)d) & 3) == 0) {
        Pack16<uint32_t> w;
        w.u = v;
#pragma unroll
        for (int k = 0; k < 4; ++k) ((uint32_t *)d)[k] = w.e[k];
        return;
    }
    Pack16<uint8_t> t;
    t.u = v;
#pragma unroll
    for (int k = 0; k < 16; ++k) d[k] = t.e[k];
}

// multicast store of a local range (bytes is a multiple of 16); a source that is not 16-byte aligned takes a slow path
static __device__ __noinline__ void pipe_copy_mc(const uint8_t *a, uint8_t *d_mc, uint64_t bytes)
{
    if (aligned16(a)) { copy_range_mc(a, d_mc, bytes); return; }
    for (uint64_t i = threadIdx.x; i < (bytes >> 4); i += blockDim.x) multimem_st_v4(d_mc + (i << 4), ld_any16(a + (i << 4)));
}
template <class T, int OP>
static __device__ __noinline__ void pipe_reduce_all(const uint8_t *const *src, int p, uint8_t *d, uint64_t n) { reduce_all_range<T, OP>(src, p, d, nullptr, n); }
template <class T, int OP>
static __device__ __noinline__ void pipe_reduce_to_all(const uint8_t *const *src, uint8_t *const *dst, int p, uint64_t n) { reduce_to_all_range<T, OP>(src, dst, p, n); }
// in-switch reduction of `bytes` (a multiple of 16) at mc into d: the multicast mapping itself, or local memory of any alignment
template <class T, int OP>
static __device__ __noinline__ void pipe_mc_reduce(const uint8_t *mc, uint8_t *d, bool d_is_mc, uint64_t bytes)
{
    if constexpr (McSupported<T, OP>::value) {
        if (d_is_mc || aligned16(d)) { mc_reduce_range<T, OP>(mc, d, d_is_mc, nullptr, bytes); return; }
        for (uint64_t i = threadIdx.x; i < (bytes >> 4); i += blockDim.x) st_any16(d + (i << 4), multimem_ld_reduce<T, OP>(mc + (i << 4)));
    }
}

template <class T, int OP>
__global__ void __launch_bounds__(kExecThreads, 1) pipe_coll_kernel(const RankCtx *ctxs, const PipeArgsArray args)
{
    const PipeArgs &a = args.a[blockIdx.y];
    const int tid = threadIdx.x, b = blockIdx.x, nb = gridDim.x;
    __shared__ RankCtx s_ctx;
    __shared__ int s_fail, s_last;
    __shared__ const uint8_t *s_src[kMaxRanks];
    __shared__ uint8_t *s_dst[kMaxRanks];
    __shared__ uint64_t s_bytes[kMaxRanks];
    {
        const uint64_t *gs = (const uint64_t *)&ctxs[blockIdx.y];
        for (int i = tid; i < (int)(sizeof(RankCtx) / 8); i += blockDim.x) ((uint64_t *)&s_ctx)[i] = gs[i];
    }
    if (tid == 0) { s_fail = 0; s_last = 0; }
    __syncthreads();
    const RankCtx &c = s_ctx;
    const int me = c.rank, p = c.nranks, es = dtype_size(a.dtype), mode = a.mode, K = a.nslots;
    WaitCtx w;
    w.deadline = global_timer_ns() + c.timeout_ns;
    w.abort = c.abort;
    w.local_fail = c.exit_counter + 1;
    const uint64_t half_off = (a.seq & 1) * c.stage_half;
    const uint64_t base = a.seq << kSeqShift;
    const uint32_t all = (1u << p) - 1u, self = 1u << me, others = all & ~self;
    const int succ = me + 1 < p ? me + 1 : 0, pred = me > 0 ? me - 1 : p - 1;
    const bool chain_last = succ == a.root;
    const bool bcast = pipe_mode_is_bcast(mode), three = pipe_mode_has_copy_out(mode);

    // ---- stage of this CTA
    int role, idx, nrole;
    if (bcast) {
        role = me == a.root ? 0 : 1; idx = b; nrole = nb;
    } else if (b < a.n1) {
        role = 0; idx = b; nrole = a.n1;
    } else if (!three || b < a.n1 + a.n2) {
        role = 1; idx = b - a.n1; nrole = three ? a.n2 : nb - a.n1;
    } else {
        role = 2; idx = b - a.n1 - a.n2; nrole = nb - a.n1 - a.n2;
    }
    const bool tr = c.trace && tid == 0 && idx == 0;
    uint64_t t_wait = 0, t_work = 0, t_sig = 0, t0 = 0;
    if (c.trace && tid == 0) atomicMin((unsigned long long *)&c.trace[0], (unsigned long long)global_timer_ns());

    // ---- the peers must have left the op that used this staging half before
    if (a.seq >= 2) {
        if (tid < p && tid != me) {
            uint64_t seen;
            int rc = wait_flag_ge(c.flags[me] + done_index(tid), a.seq - 2, w, seen);
            if (rc) { report_failure(c, a.seq, rc, -1, tid, b, a.seq - 2, seen); s_fail = rc; }
        }
        __syncthreads();
    }

    const uint64_t ce = a.chunk_elems, se = ce / (uint64_t)p;  // se: stride between the slices of a chunk in a push slot
    const uint64_t nchunks = ceil_div_u64(a.count, ce);
    const uint64_t slot_bytes = pipe_slot_bytes(mode, ce, es, p);
    const uint64_t vec = es >= 16 ? 1 : (uint64_t)(16 / es);
    uint8_t *const mine = c.stage[me];

    for (uint64_t ch = 0; ch < nchunks && !s_fail; ++ch) {
        const int slot = (int)(ch % (uint64_t)K);
        const uint64_t soff = half_off + (uint64_t)slot * slot_bytes;
        const uint64_t e0 = ch * ce;
        const uint64_t nc = a.count - e0 < ce ? a.count - e0 : ce;
        const uint64_t now = base + ch + 1, old = ch >= (uint64_t)K ? base + ch - (uint64_t)K + 1 : 0;
        // ---- what this stage waits for and what it publishes: {word, ranks}; set 0 at value wv0, set 1 always at `old`
        int ww0 = 0, ww1 = 0, sw0 = 0, sw1 = 0;
        uint32_t wm0 = 0, wm1 = 0, sm0 = 0, sm1 = 0;
        uint64_t wv0 = now;
        switch (mode) {
            case PM_AR2_MC:
                if (role == 0) { if (old) { ww0 = kPipeWordOut; wm0 = self; wv0 = old; } sw0 = kPipeWordReady; sm0 = all; }
                else if (role == 1) { ww0 = kPipeWordReady; wm0 = all; sw0 = kPipeWordDone; sm0 = all; }
                else { ww0 = kPipeWordDone; wm0 = all; sw0 = kPipeWordOut; sm0 = self; }
                break;
            case PM_AR2_PUSH:
                if (role == 0) { if (old) { ww0 = kPipeWordDone; wm0 = all; wv0 = old; } sw0 = kPipeWordReady; sm0 = all; }
                else if (role == 1) { ww0 = kPipeWordReady; wm0 = all; if (old) { ww1 = kPipeWordOut; wm1 = all; } sw0 = kPipeWordDone; sm0 = all; }
                else { ww0 = kPipeWordDone; wm0 = all; sw0 = kPipeWordOut; sm0 = all; }
                break;
            case PM_AR1_MC: case PM_AR1_PUSH: case PM_RS_MC: case PM_RS_PUSH:
                if (role == 0) { if (old) { ww0 = kPipeWordDone; wm0 = all; wv0 = old; } sw0 = kPipeWordReady; sm0 = all; }
                else { ww0 = kPipeWordReady; wm0 = all; sw0 = kPipeWordDone; sm0 = all; }
                break;
            case PM_AG_PULL: case PM_BC_MC:
                if (role == 0) { if (old) { ww0 = kPipeWordDone; wm0 = others; wv0 = old; } sw0 = kPipeWordReady; sm0 = others; }
                else if (mode == PM_AG_PULL) { ww0 = kPipeWordReady; wm0 = others; sw0 = kPipeWordDone; sm0 = others; }
                else { ww0 = kPipeWordReady; wm0 = 1u << a.root; sw0 = kPipeWordDone; sm0 = 1u << a.root; }
                break;
            default:  // PM_BC_PUSH
                if (role == 0) { if (old) { ww0 = kPipeWordDone; wm0 = 1u << succ; wv0 = old; } sw0 = kPipeWordReady; sm0 = 1u << succ; }
                else {
                    ww0 = kPipeWordReady; wm0 = 1u << pred;
                    sw1 = kPipeWordDone; sm1 = 1u << pred;
                    if (!chain_last) {
                        if (old) { ww1 = kPipeWordDone; wm1 = 1u << succ; }
                        sw0 = kPipeWordReady; sm0 = 1u << succ;
                    }
                }
                break;
        }
        // ---- wait
        if (tr) t0 = global_timer_ns();
        if (wm0 | wm1) {
            const int q = tid < 32 ? tid : tid - 32;
            const uint32_t m = tid < 32 ? wm0 : wm1;
            if (tid < 64 && q < p && ((m >> q) & 1u)) {
                const uint64_t want = tid < 32 ? wv0 : old;
                uint64_t seen;
                int rc = wait_flag_ge(c.flags[me] + flag_index(0, q, tid < 32 ? ww0 : ww1), want, w, seen);
                if (rc) { report_failure(c, a.seq, rc, (int)ch, q, b, want, seen); s_fail = rc; }
            }
            __syncthreads();
            if (s_fail) break;
        }
        if (tr) { uint64_t t1 = global_timer_ns(); t_wait += t1 - t0; t0 = t1; }
        // ---- work
        uint64_t lo, hi;
        // slice of the chunk that rank q owns in the two-shot modes: [slo(q), shi(q))
        const uint64_t per = round_up_u64(ceil_div_u64(nc, (uint64_t)p), vec);
        auto slo = [&](int q) { return per * (uint64_t)q < nc ? per * (uint64_t)q : nc; };
        auto shi = [&](int q) { return per * (uint64_t)(q + 1) < nc ? per * (uint64_t)(q + 1) : nc; };
        if (role == 0) {
            switch (mode) {
                case PM_AR2_MC: case PM_AR1_MC: case PM_AG_PULL: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (hi > lo) {
                        uint8_t *d2 = nullptr;
                        if (mode == PM_AG_PULL) {
                            d2 = a.out + ((uint64_t)me * a.count + e0 + lo) * es;
                            if (d2 == a.in + (e0 + lo) * es) d2 = nullptr;  // in place: the block is where it belongs
                        }
                        pipe_copy(a.in + (e0 + lo) * es, mine + soff + lo * es, d2, (hi - lo) * es, es);
                    }
                    break;
                }
                case PM_RS_MC: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (tid < p) {
                        s_src[tid] = a.in + ((uint64_t)tid * a.count + e0 + lo) * es;
                        s_dst[tid] = mine + soff + ((uint64_t)tid * ce + lo) * es;
                        s_bytes[tid] = (hi - lo) * es;
                    }
                    __syncthreads();
                    if (hi > lo) pipe_copy_pieces(s_src, s_dst, s_bytes, p, es);
                    break;
                }
                case PM_AR2_PUSH: case PM_RS_PUSH: {
                    // piece k goes to rank q = me + 1 + k: its slice of my chunk (AllReduce) or its block of my chunk (ReduceScatter)
                    if (tid < p - 1) {
                        const int q = me + 1 + tid < p ? me + 1 + tid : me + 1 + tid - p;
                        if (mode == PM_AR2_PUSH) {
                            chan_range(shi(q) - slo(q), es, nrole, idx, lo, hi);
                            s_src[tid] = a.in + (e0 + slo(q) + lo) * es;
                            s_dst[tid] = c.stage[q] + soff + ((uint64_t)me * se + lo) * es;
                        } else {
                            chan_range(nc, es, nrole, idx, lo, hi);
                            s_src[tid] = a.in + ((uint64_t)q * a.count + e0 + lo) * es;
                            s_dst[tid] = c.stage[q] + soff + ((uint64_t)me * ce + lo) * es;
                        }
                        s_bytes[tid] = hi > lo ? (hi - lo) * es : 0;
                    }
                    __syncthreads();
                    pipe_copy_pieces(s_src, s_dst, s_bytes, p - 1, es);
                    break;
                }
                case PM_AR1_PUSH: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (tid < p - 1) {
                        const int q = me + 1 + tid < p ? me + 1 + tid : me + 1 + tid - p;
                        s_dst[tid] = c.stage[q] + soff + ((uint64_t)me * ce + lo) * es;
                    }
                    __syncthreads();
                    if (hi > lo) pipe_copy_bcast(a.in + (e0 + lo) * es, s_dst, p - 1, (hi - lo) * es, es);
                    break;
                }
                case PM_BC_MC: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (hi > lo) pipe_copy_mc(a.in + (e0 + lo) * es, c.mc_stage + soff + lo * es, (hi - lo) * es);
                    break;
                }
                default: {  // PM_BC_PUSH, root
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (hi > lo) pipe_copy(a.in + (e0 + lo) * es, c.stage[succ] + soff + lo * es, nullptr, (hi - lo) * es, es);
                    break;
                }
            }
        } else if (role == 1) {
            switch (mode) {
                case PM_AR2_MC: {
                    chan_range(shi(me) - slo(me), es, nrole, idx, lo, hi);
                    if (hi > lo) {
                        const uint64_t off = soff + (slo(me) + lo) * es;
                        pipe_mc_reduce<T, OP>(c.mc_stage + off, c.mc_stage + off, true, (hi - lo) * es);
                    }
                    break;
                }
                case PM_AR2_PUSH: {
                    chan_range(shi(me) - slo(me), es, nrole, idx, lo, hi);
                    if (tid < p) {
                        const uint64_t mo = (e0 + slo(me) + lo) * es;
                        s_src[tid] = tid == me ? a.in + mo : mine + soff + ((uint64_t)tid * se + lo) * es;
                        s_dst[tid] = tid == me ? a.out + mo : c.stage[tid] + soff + (ce + slo(me) + lo) * es;
                    }
                    __syncthreads();
                    if (hi > lo) pipe_reduce_to_all<T, OP>(s_src, s_dst, p, hi - lo);
                    break;
                }
                case PM_AR1_MC: case PM_RS_MC: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (hi > lo) {
                        const uint64_t off = soff + ((mode == PM_RS_MC ? (uint64_t)me * ce : 0) + lo) * es;
                        pipe_mc_reduce<T, OP>(c.mc_stage + off, a.out + (e0 + lo) * es, false, (hi - lo) * es);
                    }
                    break;
                }
                case PM_AR1_PUSH: case PM_RS_PUSH: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (tid < p) {
                        const uint64_t own = ((mode == PM_RS_PUSH ? (uint64_t)me * a.count : 0) + e0 + lo) * es;
                        s_src[tid] = tid == me ? a.in + own : mine + soff + ((uint64_t)tid * ce + lo) * es;
                    }
                    __syncthreads();
                    if (hi > lo) pipe_reduce_all<T, OP>(s_src, p, a.out + (e0 + lo) * es, hi - lo);
                    break;
                }
                case PM_AG_PULL: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (hi > lo)
                        for (int i = 1; i < p; ++i) {
                            const int q = me + i < p ? me + i : me + i - p;
                            pipe_copy_deep(c.stage[q] + soff + lo * es, a.out + ((uint64_t)q * a.count + e0 + lo) * es, (hi - lo) * es, es);
                        }
                    break;
                }
                case PM_BC_MC: {
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (hi > lo) pipe_copy(mine + soff + lo * es, a.out + (e0 + lo) * es, nullptr, (hi - lo) * es, es);
                    break;
                }
                default: {  // PM_BC_PUSH: my slot -> my buffer, and on into the successor's slot
                    chan_range(nc, es, nrole, idx, lo, hi);
                    if (hi > lo) pipe_copy(mine + soff + lo * es, a.out + (e0 + lo) * es, chain_last ? nullptr : c.stage[succ] + soff + lo * es, (hi - lo) * es, es);
                    break;
                }
            }
        } else {
            // copy-out of the two-shot AllReduce; push mode: my own slice was written by the reduce stage already
            chan_range(nc, es, nrole, idx, lo, hi);
            const uint64_t roff = mode == PM_AR2_PUSH ? ce * es : 0;
            if (mode == PM_AR2_PUSH) {
                const uint64_t a0 = lo, a1 = hi < slo(me) ? hi : slo(me), b0 = lo > shi(me) ? lo : shi(me), b1 = hi;
                if (a1 > a0) pipe_copy(mine + soff + roff + a0 * es, a.out + (e0 + a0) * es, nullptr, (a1 - a0) * es, es);
                if (b1 > b0) pipe_copy(mine + soff + roff + b0 * es, a.out + (e0 + b0) * es, nullptr, (b1 - b0) * es, es);
            } else if (hi > lo) {
                pipe_copy(mine + soff + lo * es, a.out + (e0 + lo) * es, nullptr, (hi - lo) * es, es);
            }
        }
        if (tr) { uint64_t t1 = global_timer_ns(); t_work += t1 - t0; t0 = t1; }
        // ---- arrive; the last CTA of the stage publishes the chunk
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            uint32_t *cnt = c.pipe_cnt + role * kPipeMaxSlots + slot;
            const unsigned prev = nrole > 1 ? atomicAdd(cnt, 1u) : 0u;
            const int last = prev == (unsigned)(nrole - 1);
            if (last && nrole > 1) { atomicExch(cnt, 0u); __threadfence(); }
            s_last = last;
        }
        __syncthreads();
        if (s_last && tid < 64) {
            const int q = tid < 32 ? tid : tid - 32;
            const uint32_t m = tid < 32 ? sm0 : sm1;
            if (q < p && ((m >> q) & 1u)) st_release_sys(c.flags[q] + flag_index(0, me, tid < 32 ? sw0 : sw1), now);
        }
        if (tr) { uint64_t t1 = global_timer_ns(); t_sig += t1 - t0; }
    }
    if (tr) {
        c.trace[1 + role * 4] = t_wait; c.trace[2 + role * 4] = t_work; c.trace[3 + role * 4] = t_sig; c.trace[4 + role * 4] = global_timer_ns();
    }
    if (c.trace && tid == 0) atomicMax((unsigned long long *)&c.trace[kTraceWords - 1], (unsigned long long)global_timer_ns());
    // ---- completion: the last CTA of this rank tells every peer that this op no longer touches their memory
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        unsigned prev = atomicAdd(c.exit_counter, 1u);
        s_last = prev == gridDim.x - 1;
        if (s_last) *c.exit_counter = 0;
    }
    __syncthreads();
    if (s_last && !s_fail && *(volatile uint32_t *)(c.exit_counter + 1) == 0u) {
        if (tid < p && tid != me) st_release_sys(c.flags[tid] + done_index(me), a.seq);
        if (tid == 0) *c.dev_tail = a.seq;
    }
}

// Defines pipe_kernel_<name>(op): the pipelined kernel for element type T and reduction `op`.
#define HCCLB_INSTANTIATE_PIPE(T, name)                                                          \
    const void *pipe_kernel_##name(int op)                                                       \
    {                                                                                            \
        switch (op) {                                                                            \
            case HCCL_REDUCE_SUM: return (const void *)pipe_coll_kernel<T, HCCL_REDUCE_SUM>;     \
            case HCCL_REDUCE_PROD: return (const void *)pipe_coll_kernel<T, HCCL_REDUCE_PROD>;   \
            case HCCL_REDUCE_MAX: return (const void *)pipe_coll_kernel<T, HCCL_REDUCE_MAX>;     \
            default: return (const void *)pipe_coll_kernel<T, HCCL_REDUCE_MIN>;                  \
        }                                                                                        \
    }

}  // namespace hcclb
