// Pipelined large-message kernel for sm_100a: see pipe_coll.h for the role it plays.  One kernel per (element type,
// reduction operator), instantiated next to the plan executor of the same type.
//
// Protocol.  The op's half of the staging buffer is a ring of `nslots` slots; chunk c lives in slot c % nslots on every
// rank.  The CTAs of a rank form up to three stages, and a stage may split into groups that take chunks in turn (group g
// of G works on the chunks c with c % G == g), so that one group's flag traffic hides behind another group's transfer.
// Every CTA of a group works on its share of the group's chunk; when it is done it adds one to that slot's arrival
// counter (gpu scope), and the CTA that arrives last publishes the stage's progress on that slot, (seq << kSeqShift) +
// c + 1, with ONE st.release.sys per destination rank (its own page included, for the next stage of the same rank).
// Progress words are kept per (stage, source rank, slot): a stage starts chunk c when the words it depends on have
// reached c + 1 for that slot, and it writes into a slot again only after every reader of the chunk that lived there
// has published, so the ring needs no other hand-shake.  Every dependency points to an earlier stage of the same chunk
// or to an earlier chunk, so the stages cannot wait on one another in a cycle.  All waits are bounded (wait_flag_ge,
// mbarrier polls with an iteration limit); a CTA that gives up records the status block and every other CTA of the
// rank leaves at its next wait.
//
// Data movement.  Plain copies (stage-in, push to the peers' slots, pull from the peers' slots, copy-out) are driven
// by one thread per CTA with bulk asynchronous copies (cp.async.bulk global -> shared -> global, never multicast)
// through a 6 x 32 KB shared-memory ring: 160 KB in flight per SM without a register, which is what a microsecond-scale
// NVLink round trip needs.  The reductions of the push modes are fed the same way: thread 0 streams tiles of the p
// sources into the ring, all threads reduce a stage from shared memory in registers and store the result straight to
// its destinations.  The in-switch modes reduce with multimem.ld_reduce / multimem.st in registers.  Buffers that are
// not 16-byte aligned take plain register loops instead.
#pragma once
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.h"

namespace hcclb {

constexpr uint32_t kPipeSpin = 1u << 26;  // polls of an mbarrier before the driver thread gives up (seconds)
constexpr int kPipeSegs = 2 * kMaxRanks;

namespace pipe_detail {
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    for (uint32_t it = 0; it < kPipeSpin; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *dst, const void *src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
}  // namespace pipe_detail

// nseg independent copies (segment k: bytes[k] from src[k] to dst[k]; all 16-byte aligned, sizes multiples of 16) by bulk
// asynchronous copies through the shared-memory ring; loads run kTmaDepth - 1 pieces ahead of the stores.  Called by ONE
// thread.  `g` counts pieces over the kernel's lifetime (ring slot = g % depth, mbarrier parity = (g / depth) & 1).  On
// return every store has completed and is ordered before the caller's later generic-proxy accesses.  False: an mbarrier
// poll ran out (the loads still in flight are given the same bound to land before the caller leaves).
static __device__ __noinline__ bool tma_copy_segments(uint8_t *ring, uint64_t *bar, uint32_t &g, int nseg, const uint8_t *const *src,
                                                      uint8_t *const *dst, const uint64_t *bytes)
{
    using namespace pipe_detail;
    uint32_t loaded = 0, stored = 0;
    int lk = 0, sk = 0;
    uint64_t loff = 0, soff = 0;
    while (lk < nseg && loff >= bytes[lk]) { ++lk; loff = 0; }
    while (sk < nseg && soff >= bytes[sk]) { ++sk; soff = 0; }
    auto issue_load = [&]() {
        const uint64_t left = bytes[lk] - loff;
        const uint32_t len = left < kTmaBuf ? (uint32_t)left : kTmaBuf, slot = (g + loaded) % kTmaDepth;
        mbar_expect_tx(&bar[slot], len);
        bulk_g2s(ring + (size_t)slot * kTmaBuf, src[lk] + loff, len, &bar[slot]);
        loff += len;
        ++loaded;
        while (lk < nseg && loff >= bytes[lk]) { ++lk; loff = 0; }
    };
    fence_proxy_async();  // what other threads and ranks wrote with ordinary stores is read by the copy engine from here on
    while (lk < nseg && loaded < (uint32_t)(kTmaDepth - 1)) issue_load();
    bool ok = true;
    while (sk < nseg) {
        const uint32_t idx = g + stored, slot = idx % kTmaDepth;
        if (!mbar_wait(&bar[slot], (idx / kTmaDepth) & 1)) { ok = false; break; }
        const uint64_t left = bytes[sk] - soff;
        const uint32_t len = left < kTmaBuf ? (uint32_t)left : kTmaBuf;
        bulk_s2g(dst[sk] + soff, ring + (size_t)slot * kTmaBuf, len);
        bulk_commit();
        soff += len;
        ++stored;
        while (sk < nseg && soff >= bytes[sk]) { ++sk; soff = 0; }
        bulk_wait_read<1>();  // the store before this one has read its ring slot: that slot takes the next load
        if (lk < nseg) issue_load();
    }
    if (!ok)
        for (uint32_t i = stored; i < loaded; ++i) mbar_wait(&bar[(g + i) % kTmaDepth], ((g + i) / kTmaDepth) & 1);
    g += loaded;
    bulk_wait_all<0>();
    fence_proxy_async();
    return ok;
}

// The register loops are kept out of line: each gets its own register allocation, and the stage loop stays small.
// nseg independent copies of any alignment; two vectors of each of eight segments in flight per thread on the aligned path
static __device__ __noinline__ void pipe_copy_segments(const uint8_t *const *src, uint8_t *const *dst, const uint64_t *bytes, int nseg, int es)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    bool fast = true;
    uint64_t mx = 0;
    for (int k = 0; k < nseg; ++k) {
        fast = fast && aligned16(src[k]) && aligned16(dst[k]) && (bytes[k] & 15) == 0;
        mx = bytes[k] > mx ? bytes[k] : mx;
    }
    if (!fast) {
        for (int k = 0; k < nseg; ++k)
            if (bytes[k]) copy_range(src[k], dst[k], nullptr, bytes[k], es);
        return;
    }
    const uint64_t nvec = mx >> 4;
    for (int k0 = 0; k0 < nseg; k0 += 8) {
        for (uint64_t i = tid; i < nvec; i += 2ull * nt) {
            uint4 v[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k0 + k < nseg && ((i + (uint64_t)u * nt) << 4) < bytes[k0 + k]) v[u][k] = ld_stream((const uint4 *)src[k0 + k] + i + (uint64_t)u * nt);
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (k0 + k < nseg && ((i + (uint64_t)u * nt) << 4) < bytes[k0 + k]) ((uint4 *)dst[k0 + k])[i + (uint64_t)u * nt] = v[u][k];
        }
    }
}

__device__ __forceinline__ uint4 ld_any16(const uint8_t *a)
{
    if ((((uintptr_t)a) & 3) == 0) {
        Pack16<uint32_t> w;
#pragma unroll
        for (int k = 0; k < 4; ++k) w.e[k] = ((const uint32_t *)a)[k];
        return w.u;
    }
    Pack16<uint8_t> t;
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

// dst[q] (q < nd) = reduction over the p <= NP sources in rank order; U vectors of every source in flight per thread.
template <class T, int OP, int NP, int U>
__device__ __forceinline__ void reduce_vec(const uint8_t *const *src, int p, uint8_t *const *dst, int nd, uint64_t nvec)
{
    using N = DNum<T>;
    using Acc = typename N::Acc;
    constexpr int E = 16 / sizeof(T);
    const int tid = threadIdx.x, nt = blockDim.x;
    for (uint64_t i = tid; i < nvec; i += (uint64_t)U * nt) {
        uint4 v[U][NP];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int q = 0; q < NP; ++q)
                if (q < p && i + (uint64_t)u * nt < nvec) v[u][q] = ld_stream((const uint4 *)src[q] + i + (uint64_t)u * nt);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t idx = i + (uint64_t)u * nt;
            if (idx < nvec) {
                Acc acc[E];
                Pack16<T> t;
                t.u = v[u][0];
#pragma unroll
                for (int k = 0; k < E; ++k) acc[k] = N::up(t.e[k]);
#pragma unroll
                for (int q = 1; q < NP; ++q)
                    if (q < p) {
                        Pack16<T> y;
                        y.u = v[u][q];
#pragma unroll
                        for (int k = 0; k < E; ++k) acc[k] = red_op<OP>(acc[k], N::up(y.e[k]));
                    }
                Pack16<T> z;
#pragma unroll
                for (int k = 0; k < E; ++k) z.e[k] = N::down(acc[k]);
                for (int q = 0; q < nd; ++q) ((uint4 *)dst[q])[idx] = z.u;
            }
        }
    }
}

// dst[q] (q < nd) = reduction of n elements over the p sources in rank order (fixed order: every rank computes the same bits)
template <class T, int OP>
static __device__ __noinline__ void pipe_reduce(const uint8_t *const *src, int p, uint8_t *const *dst, int nd, uint64_t n)
{
    using N = DNum<T>;
    using Acc = typename N::Acc;
    constexpr int E = 16 / sizeof(T);
    bool al = p <= 8;
    for (int q = 0; q < p; ++q) al = al && aligned16(src[q]);
    for (int q = 0; q < nd; ++q) al = al && aligned16(dst[q]);
    uint64_t done = 0;
    if (al) {
        const uint64_t nvec = n / E;
        if (p <= 2) reduce_vec<T, OP, 2, 4>(src, p, dst, nd, nvec);
        else if (p <= 4) reduce_vec<T, OP, 4, 2>(src, p, dst, nd, nvec);
        else reduce_vec<T, OP, 8, 1>(src, p, dst, nd, nvec);
        done = nvec * E;
    }
    for (uint64_t i = done + threadIdx.x; i < n; i += blockDim.x) {
        Acc acc = N::up(((const T *)src[0])[i]);
        for (int q = 1; q < p; ++q) acc = red_op<OP>(acc, N::up(((const T *)src[q])[i]));
        const T v = N::down(acc);
        for (int q = 0; q < nd; ++q) ((T *)dst[q])[i] = v;
    }
}

// Same reduction fed by the copy engine: thread 0 streams tiles of the p sources into the shared-memory ring with bulk
// asynchronous copies (kStages - 1 stages ahead, about 160 KB in flight), all threads reduce a stage from shared memory in
// registers and store the result straight to the nd destinations.  All addresses 16-byte aligned, `bytes` a multiple of 16,
// p <= NP.  `g` counts stages over the kernel's lifetime (as in tma_copy_segments; a CTA uses one of the two, never both).
// False: an mbarrier poll ran out.
template <class T, int OP, int NP>
__device__ __forceinline__ bool tma_reduce_np(uint8_t *ring, uint64_t *bar, uint32_t &g, const uint8_t *const *src, int p, uint8_t *const *dst,
                                             int nd, uint64_t bytes)
{
    using namespace pipe_detail;
    using N = DNum<T>;
    using Acc = typename N::Acc;
    constexpr int E = 16 / sizeof(T);
    constexpr uint32_t kStageBytes = NP == 8 ? 2 * kTmaBuf : kTmaBuf;       // p tiles per stage
    constexpr int kStages = (int)(kPipeDynSmem / kStageBytes);
    constexpr uint32_t kTile = kStageBytes / NP;
    const int tid = threadIdx.x, nt = blockDim.x;
    const uint64_t ntiles = (bytes + kTile - 1) / kTile;
    auto issue = [&](uint64_t t) {
        const uint64_t off = t * kTile;
        const uint32_t len = bytes - off < kTile ? (uint32_t)(bytes - off) : kTile, st = (uint32_t)((g + t) % kStages);
        mbar_expect_tx(&bar[st], len * (uint32_t)p);
        for (int q = 0; q < p; ++q) bulk_g2s(ring + (size_t)st * kStageBytes + (size_t)q * kTile, src[q] + off, len, &bar[st]);
    };
    if (tid == 0) {
        fence_proxy_async();
        for (uint64_t t = 0; t < ntiles && t < (uint64_t)(kStages - 1); ++t) issue(t);
    }
    bool ok = true;
    for (uint64_t t = 0; t < ntiles; ++t) {
        if (tid == 0 && t + kStages - 1 < ntiles) issue(t + kStages - 1);  // into the stage that tile t - 1 left at the barrier below
        const uint32_t st = (uint32_t)((g + t) % kStages);
        if (!mbar_wait(&bar[st], (uint32_t)(((g + t) / kStages) & 1))) { ok = false; break; }
        const uint64_t off = t * kTile;
        const uint32_t nv = (uint32_t)((bytes - off < kTile ? bytes - off : kTile) >> 4);
        const uint4 *tile = (const uint4 *)(ring + (size_t)st * kStageBytes);
        for (uint32_t i = tid; i < nv; i += nt) {
            Pack16<T> x;
            x.u = tile[i];
            Acc acc[E];
#pragma unroll
            for (int k = 0; k < E; ++k) acc[k] = N::up(x.e[k]);
#pragma unroll
            for (int q = 1; q < NP; ++q)
                if (q < p) {
                    Pack16<T> y;
                    y.u = tile[(size_t)q * (kTile >> 4) + i];
#pragma unroll
                    for (int k = 0; k < E; ++k) acc[k] = red_op<OP>(acc[k], N::up(y.e[k]));
                }
            Pack16<T> z;
#pragma unroll
            for (int k = 0; k < E; ++k) z.e[k] = N::down(acc[k]);
            for (int q = 0; q < nd; ++q) ((uint4 *)(dst[q] + off))[i] = z.u;
        }
        __syncthreads();  // every thread has read the stage: it may be loaded again
    }
    g += (uint32_t)ntiles;
    return ok;
}
template <class T, int OP>
static __device__ __noinline__ bool tma_reduce(uint8_t *ring, uint64_t *bar, uint32_t &g, const uint8_t *const *src, int p, uint8_t *const *dst, int nd,
                                               uint64_t bytes)
{
    if (p <= 2) return tma_reduce_np<T, OP, 2>(ring, bar, g, src, p, dst, nd, bytes);
    if (p <= 4) return tma_reduce_np<T, OP, 4>(ring, bar, g, src, p, dst, nd, bytes);
    return tma_reduce_np<T, OP, 8>(ring, bar, g, src, p, dst, nd, bytes);
}

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
    using namespace pipe_detail;
    extern __shared__ __align__(128) uint8_t pipe_ring[];
    const PipeArgs &a = args.a[blockIdx.y];
    const int tid = threadIdx.x, b = blockIdx.x, nb = gridDim.x;
    __shared__ RankCtx s_ctx;
    __shared__ int s_fail, s_last;
    __shared__ const uint8_t *s_src[kPipeSegs];
    __shared__ uint8_t *s_dst[kPipeSegs];
    __shared__ uint64_t s_bytes[kPipeSegs];
    __shared__ __align__(8) uint64_t s_bar[kTmaDepth];
    {
        const uint64_t *gs = (const uint64_t *)&ctxs[blockIdx.y];
        for (int i = tid; i < (int)(sizeof(RankCtx) / 8); i += blockDim.x) ((uint64_t *)&s_ctx)[i] = gs[i];
    }
    if (tid == 0) {
        s_fail = 0;
        s_last = 0;
        for (int i = 0; i < kTmaDepth; ++i) mbar_init(&s_bar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
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
    uint32_t tma_g = 0;  // pieces this CTA's driver thread has pushed through the ring (thread 0 only)

    // ---- stage and group of this CTA
    int role, idx, nrole, ngroup;
    if (bcast) {
        role = me == a.root ? 0 : 1; idx = b; nrole = nb; ngroup = a.g1;
    } else if (b < a.n1) {
        role = 0; idx = b; nrole = a.n1; ngroup = a.g1;
    } else if (!three || b < a.n1 + a.n2) {
        role = 1; idx = b - a.n1; nrole = three ? a.n2 : nb - a.n1; ngroup = a.g2;
    } else {
        role = 2; idx = b - a.n1 - a.n2; nrole = nb - a.n1 - a.n2; ngroup = a.g3;
    }
    if (ngroup < 1 || nrole % ngroup != 0) ngroup = 1;
    const int group = idx % ngroup, gidx = idx / ngroup, gsize = nrole / ngroup;
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

    // copies the segments described in s_src / s_dst / s_bytes: by the copy engine when everything is 16-byte aligned
    auto copy_segments = [&](int nseg) {
        bool tma = true;
        for (int k = 0; k < nseg; ++k) tma = tma && aligned16(s_src[k]) && aligned16(s_dst[k]) && (s_bytes[k] & 15) == 0;
        if (!tma) { pipe_copy_segments(s_src, s_dst, s_bytes, nseg, es); return; }
        if (tid == 0 && !tma_copy_segments(pipe_ring, s_bar, tma_g, nseg, s_src, s_dst, s_bytes)) {
            report_failure(c, a.seq, HCCL_E_TIMEOUT, -2, me, b, 0, 0);
            s_fail = HCCL_E_TIMEOUT;
        }
    };

    // dst[0..nd) = reduction of n elements over the p sources in s_src: fed by the copy engine when everything is aligned
    auto reduce_sources = [&](int nd, uint64_t n) {
        bool tma = p <= 8 && ((n * es) & 15) == 0;
        for (int q = 0; q < p; ++q) tma = tma && aligned16(s_src[q]);
        for (int q = 0; q < nd; ++q) tma = tma && aligned16(s_dst[q]);
        if (!tma) { if (n) pipe_reduce<T, OP>(s_src, p, s_dst, nd, n); return; }
        if (!tma_reduce<T, OP>(pipe_ring, s_bar, tma_g, s_src, p, s_dst, nd, n * es) && tid == 0) {
            report_failure(c, a.seq, HCCL_E_TIMEOUT, -3, me, b, 0, 0);
            s_fail = HCCL_E_TIMEOUT;
        }
    };

    if (pipe_mode_is_zc(mode)) {
        // ---- zero-copy modes: no staging, one round.  Flag words of slot 0 carry the hand-shake.
        const uint64_t now = base + 1;
        if (role == 0) {
            // gate: this rank's send buffer is complete (stream order) and may be read; then hold the kernel, and with it
            // everything the caller enqueues behind it, until every peer has finished reading
            if (tid < p && tid != me) st_release_sys(c.flags[tid] + pipe_flag_index(kPipeWordReady, me, 0), now);
            if (tid < p && tid != me) {
                uint64_t seen;
                int rc = wait_flag_ge(c.flags[me] + pipe_flag_index(kPipeWordDone, tid, 0), now, w, seen);
                if (rc) { report_failure(c, a.seq, rc, 1, tid, b, now, seen); s_fail = rc; }
            }
        } else {
            if (tid < p && tid != me) {
                uint64_t seen;
                int rc = wait_flag_ge(c.flags[me] + pipe_flag_index(kPipeWordReady, tid, 0), now, w, seen);
                if (rc) { report_failure(c, a.seq, rc, 0, tid, b, now, seen); s_fail = rc; }
            }
            __syncthreads();
            if (!s_fail) {
                uint64_t lo, hi;
                chan_range(a.count, es, nrole, idx, lo, hi);
                auto peer_in = [&](int q) { return q == me ? a.in : a.z_in_peer[q] + a.z_in_off; };
                if (mode == PM_AG_ZC) {
                    if (tid < p) {
                        const int q = me + tid < p ? me + tid : me + tid - p;  // segment 0 is my own block
                        s_src[tid] = peer_in(q) + lo * es;
                        s_dst[tid] = a.out + ((uint64_t)q * a.count + lo) * es;
                        s_bytes[tid] = hi > lo && !(q == me && s_dst[tid] == s_src[tid]) ? (hi - lo) * es : 0;
                    }
                    __syncthreads();
                    copy_segments(p);
                } else {
                    if (tid < p) s_src[tid] = peer_in(tid) + ((mode == PM_RS_ZC ? (uint64_t)me * a.count : 0) + lo) * es;
                    if (tid == 0) s_dst[0] = a.out + lo * es;
                    __syncthreads();
                    reduce_sources(1, hi > lo ? hi - lo : 0);
                }
            }
            // the last CTA of the stage tells the peers that this rank has finished reading their buffers
            __syncthreads();
            if (tid == 0) {
                __threadfence();
                uint32_t *cnt = c.pipe_cnt + kPipeMaxSlots;
                const unsigned prev = nrole > 1 ? atomicAdd(cnt, 1u) : 0u;
                const int last = prev == (unsigned)(nrole - 1);
                if (last && nrole > 1) { atomicExch(cnt, 0u); __threadfence(); }
                s_last = last;
            }
            __syncthreads();
            if (s_last && !s_fail && tid < p && tid != me) st_release_sys(c.flags[tid] + pipe_flag_index(kPipeWordDone, me, 0), now);
        }
    }
    // Reduce: every rank but the root owns a slice of each chunk (two ranks: the root owns all of it), so that the root only
    // takes in reduced slices: one message's worth of bytes over each rank's links in each direction.  Owner k is rank
    // rd_owner(k); an owner's slot holds the slices of its p - 1 sources, rd_se elements apart.
    const int rd_nown = p == 2 ? 1 : p - 1;
    auto rd_owner = [&](int k) { return p == 2 ? (int)a.root : (a.root + 1 + k < p ? a.root + 1 + k : a.root + 1 + k - p); };
    const int rd_mine = p == 2 ? (me == a.root ? 0 : -1) : (me == a.root ? -1 : (me > a.root ? me - a.root - 1 : me + p - a.root - 1));
    const uint64_t rd_se = ce / (uint64_t)rd_nown;
    // only the root has a receive buffer, the copy-out CTAs of the other ranks have nothing to do
    const bool idle = pipe_mode_is_zc(mode) || (mode == PM_RD_PUSH && role == 2 && me != a.root);
    for (uint64_t ch = (uint64_t)group; ch < nchunks && !s_fail && !idle; ch += (uint64_t)ngroup) {
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
            case PM_RD_PUSH: {
                const uint32_t rootm = 1u << a.root;
                if (role == 0) { if (old) { ww0 = kPipeWordDone; wm0 = all; wv0 = old; } sw0 = kPipeWordReady; sm0 = all; }
                else if (role == 1) { ww0 = kPipeWordReady; wm0 = all; if (old) { ww1 = kPipeWordOut; wm1 = rootm; } sw0 = kPipeWordDone; sm0 = all; }
                else { ww0 = kPipeWordDone; wm0 = all; sw0 = kPipeWordOut; sm0 = all; }  // the root only (see the loop bound)
                break;
            }
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
                int rc = wait_flag_ge(c.flags[me] + pipe_flag_index(tid < 32 ? ww0 : ww1, q, slot), want, w, seen);
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
        // Reduce: the slices of a chunk belong to the owners (rd_nown of them), slice k = [rd_lo(k), rd_hi(k))
        const uint64_t rd_per = round_up_u64(ceil_div_u64(nc, (uint64_t)rd_nown), vec);
        auto rd_lo = [&](int k) { return rd_per * (uint64_t)k < nc ? rd_per * (uint64_t)k : nc; };
        auto rd_hi = [&](int k) { return rd_per * (uint64_t)(k + 1) < nc ? rd_per * (uint64_t)(k + 1) : nc; };
        if (role == 0) {
            int nseg = 1;
            switch (mode) {
                case PM_AR2_MC: case PM_AR1_MC: case PM_AG_PULL: case PM_BC_PUSH: {
                    chan_range(nc, es, gsize, gidx, lo, hi);
                    if (tid == 0) {
                        s_src[0] = a.in + (e0 + lo) * es;
                        s_dst[0] = (mode == PM_BC_PUSH ? c.stage[succ] : mine) + soff + lo * es;
                        s_bytes[0] = (hi - lo) * es;
                        // AllGather: my own block also goes straight to its place in my receive buffer (unless it is there already)
                        s_src[1] = s_src[0];
                        s_dst[1] = a.out + ((uint64_t)me * a.count + e0 + lo) * es;
                        s_bytes[1] = s_bytes[0];
                    }
                    if (mode == PM_AG_PULL && a.out + (uint64_t)me * a.count * es != a.in) nseg = 2;
                    break;
                }
                case PM_RS_MC: {
                    chan_range(nc, es, gsize, gidx, lo, hi);
                    if (tid < p) {
                        s_src[tid] = a.in + ((uint64_t)tid * a.count + e0 + lo) * es;
                        s_dst[tid] = mine + soff + ((uint64_t)tid * ce + lo) * es;
                        s_bytes[tid] = (hi - lo) * es;
                    }
                    nseg = p;
                    break;
                }
                case PM_RD_PUSH: {
                    // my slice for owner k goes into that owner's slot, at my position among its p - 1 sources
                    nseg = rd_nown - (rd_mine >= 0 ? 1 : 0);
                    if (tid < nseg) {
                        const int k = rd_mine >= 0 && tid >= rd_mine ? tid + 1 : tid;  // owners but me
                        const int q = rd_owner(k);
                        chan_range(rd_hi(k) - rd_lo(k), es, gsize, gidx, lo, hi);
                        s_src[tid] = a.in + (e0 + rd_lo(k) + lo) * es;
                        s_dst[tid] = c.stage[q] + soff + ((uint64_t)(me < q ? me : me - 1) * rd_se + lo) * es;
                        s_bytes[tid] = hi > lo ? (hi - lo) * es : 0;
                    }
                    break;
                }
                case PM_AR2_PUSH: case PM_RS_PUSH: case PM_AR1_PUSH: {
                    // segment k goes to rank q = me + 1 + k: its slice of my chunk (two-shot), its block of my chunk
                    // (ReduceScatter), or the whole chunk (one-shot)
                    if (tid < p - 1) {
                        const int q = me + 1 + tid < p ? me + 1 + tid : me + 1 + tid - p;
                        if (mode == PM_AR2_PUSH) {
                            chan_range(shi(q) - slo(q), es, gsize, gidx, lo, hi);
                            s_src[tid] = a.in + (e0 + slo(q) + lo) * es;
                            s_dst[tid] = c.stage[q] + soff + ((uint64_t)me * se + lo) * es;
                        } else {
                            chan_range(nc, es, gsize, gidx, lo, hi);
                            s_src[tid] = a.in + ((mode == PM_RS_PUSH ? (uint64_t)q * a.count : 0) + e0 + lo) * es;
                            s_dst[tid] = c.stage[q] + soff + ((uint64_t)me * ce + lo) * es;
                        }
                        s_bytes[tid] = hi > lo ? (hi - lo) * es : 0;
                    }
                    nseg = p - 1;
                    break;
                }
                default: {  // PM_BC_MC
                    nseg = 0;
                    chan_range(nc, es, gsize, gidx, lo, hi);
                    if (hi > lo) pipe_copy_mc(a.in + (e0 + lo) * es, c.mc_stage + soff + lo * es, (hi - lo) * es);
                    break;
                }
            }
            if (nseg) {
                __syncthreads();
                copy_segments(nseg);
            }
        } else if (role == 1) {
            switch (mode) {
                case PM_AR2_MC: {
                    chan_range(shi(me) - slo(me), es, gsize, gidx, lo, hi);
                    if (hi > lo) {
                        const uint64_t off = soff + (slo(me) + lo) * es;
                        pipe_mc_reduce<T, OP>(c.mc_stage + off, c.mc_stage + off, true, (hi - lo) * es);
                    }
                    break;
                }
                case PM_AR2_PUSH: {
                    chan_range(shi(me) - slo(me), es, gsize, gidx, lo, hi);
                    if (tid < p) {
                        const uint64_t mo = (e0 + slo(me) + lo) * es;
                        s_src[tid] = tid == me ? a.in + mo : mine + soff + ((uint64_t)tid * se + lo) * es;
                        s_dst[tid] = tid == me ? a.out + mo : c.stage[tid] + soff + (ce + slo(me) + lo) * es;
                    }
                    __syncthreads();
                    reduce_sources(p, hi > lo ? hi - lo : 0);
                    break;
                }
                case PM_RD_PUSH: {
                    if (rd_mine < 0) break;  // not an owner: nothing to reduce (the stage still publishes, for the slot bookkeeping)
                    chan_range(rd_hi(rd_mine) - rd_lo(rd_mine), es, gsize, gidx, lo, hi);
                    if (tid < p) {
                        const uint64_t mo = (e0 + rd_lo(rd_mine) + lo) * es;
                        s_src[tid] = tid == me ? a.in + mo : mine + soff + ((uint64_t)(tid < me ? tid : tid - 1) * rd_se + lo) * es;
                        if (tid == 0) s_dst[0] = me == a.root ? a.out + mo : c.stage[a.root] + soff + (ce + rd_lo(rd_mine) + lo) * es;
                    }
                    __syncthreads();
                    reduce_sources(1, hi > lo ? hi - lo : 0);
                    break;
                }
                case PM_AR1_MC: case PM_RS_MC: {
                    chan_range(nc, es, gsize, gidx, lo, hi);
                    if (hi > lo) {
                        const uint64_t off = soff + ((mode == PM_RS_MC ? (uint64_t)me * ce : 0) + lo) * es;
                        pipe_mc_reduce<T, OP>(c.mc_stage + off, a.out + (e0 + lo) * es, false, (hi - lo) * es);
                    }
                    break;
                }
                case PM_AR1_PUSH: case PM_RS_PUSH: {
                    chan_range(nc, es, gsize, gidx, lo, hi);
                    if (tid < p) {
                        const uint64_t own = ((mode == PM_RS_PUSH ? (uint64_t)me * a.count : 0) + e0 + lo) * es;
                        s_src[tid] = tid == me ? a.in + own : mine + soff + ((uint64_t)tid * ce + lo) * es;
                        if (tid == 0) s_dst[0] = a.out + (e0 + lo) * es;
                    }
                    __syncthreads();
                    reduce_sources(1, hi > lo ? hi - lo : 0);
                    break;
                }
                case PM_AG_PULL: {
                    chan_range(nc, es, gsize, gidx, lo, hi);
                    if (tid < p - 1) {
                        const int q = me + 1 + tid < p ? me + 1 + tid : me + 1 + tid - p;
                        s_src[tid] = c.stage[q] + soff + lo * es;
                        s_dst[tid] = a.out + ((uint64_t)q * a.count + e0 + lo) * es;
                        s_bytes[tid] = (hi - lo) * es;
                    }
                    __syncthreads();
                    copy_segments(p - 1);
                    break;
                }
                default: {  // PM_BC_MC, PM_BC_PUSH: my slot -> my buffer (push: and on into the successor's slot)
                    chan_range(nc, es, gsize, gidx, lo, hi);
                    if (tid == 0) {
                        s_src[0] = s_src[1] = mine + soff + lo * es;
                        s_dst[0] = a.out + (e0 + lo) * es;
                        s_dst[1] = c.stage[succ] + soff + lo * es;
                        s_bytes[0] = s_bytes[1] = (hi - lo) * es;
                    }
                    __syncthreads();
                    copy_segments(mode == PM_BC_PUSH && !chain_last ? 2 : 1);
                    break;
                }
            }
        } else {
            // copy-out of the two-shot AllReduce; push mode: my own slice was written by the reduce stage already
            chan_range(nc, es, gsize, gidx, lo, hi);
            if (tid == 0) {
                const bool push = mode == PM_AR2_PUSH || mode == PM_RD_PUSH;
                const uint64_t roff = push ? ce * es : 0;
                // what the reduce stage of this rank wrote straight to the receive buffer: its own slice
                uint64_t own_lo = slo(me), own_hi = shi(me);
                if (mode == PM_RD_PUSH) { own_lo = rd_mine >= 0 ? rd_lo(rd_mine) : 0; own_hi = rd_mine >= 0 ? rd_hi(rd_mine) : 0; }
                uint64_t a0 = lo, a1 = hi, b0 = hi, b1 = hi;
                if (push) { a1 = hi < own_lo ? hi : own_lo; b0 = lo > own_hi ? lo : own_hi; if (a1 < a0) a1 = a0; }
                s_src[0] = mine + soff + roff + a0 * es; s_dst[0] = a.out + (e0 + a0) * es; s_bytes[0] = a1 > a0 ? (a1 - a0) * es : 0;
                s_src[1] = mine + soff + roff + b0 * es; s_dst[1] = a.out + (e0 + b0) * es; s_bytes[1] = b1 > b0 ? (b1 - b0) * es : 0;
            }
            __syncthreads();
            copy_segments(2);
        }
        if (tr) { uint64_t t1 = global_timer_ns(); t_work += t1 - t0; t0 = t1; }
        // ---- arrive; the last CTA of the group publishes the chunk
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            uint32_t *cnt = c.pipe_cnt + role * kPipeMaxSlots + slot;
            const unsigned prev = gsize > 1 ? atomicAdd(cnt, 1u) : 0u;
            const int last = prev == (unsigned)(gsize - 1);
            if (last && gsize > 1) { atomicExch(cnt, 0u); __threadfence(); }
            s_last = last;
        }
        __syncthreads();
        if (s_last && tid < 64 && !s_fail) {
            const int q = tid < 32 ? tid : tid - 32;
            const uint32_t m = tid < 32 ? sm0 : sm1;
            if (q < p && ((m >> q) & 1u)) st_release_sys(c.flags[q] + pipe_flag_index(tid < 32 ? sw0 : sw1, me, slot), now);
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
