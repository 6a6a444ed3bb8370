// Templated device executor: see exec_plan.cu for the description.  One kernel per (element type, reduction operator)
// is instantiated in its own translation unit (exec_plan_<type>.cu) so that every kernel is small: the reduction is
// resolved at compile time, nothing is dispatched inside the kernel and the typed loops keep their data in registers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <type_traits>
#include "algo/plan.h"
#include "algo/resolve.h"
#include "kernels/prims.cuh"

namespace hcclb {

constexpr int kExecThreads = 512;
constexpr int kSmemSteps = 96;  // steps of a plan kept in shared memory (longer plans read the rest from global memory)

struct ExecArgsArray {
    ExecArgs a[kMaxRanks];
};

// ---------------------------------------------------------------------------------------------- numerics
template <class T> struct DNum { using Acc = T; static __device__ __forceinline__ Acc up(T v) { return v; } static __device__ __forceinline__ T down(Acc v) { return v; } };
template <> struct DNum<__half> { using Acc = float; static __device__ __forceinline__ float up(__half v) { return __half2float(v); } static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); } };
template <> struct DNum<__nv_bfloat16> { using Acc = float; static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); } static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); } };

template <int OP, class A> __device__ __forceinline__ A red_op(A x, A y)
{
    if (OP == HCCL_REDUCE_SUM) return (A)(x + y);
    if (OP == HCCL_REDUCE_PROD) return (A)(x * y);
    if (OP == HCCL_REDUCE_MAX) return x > y ? x : y;
    return x < y ? x : y;
}

template <class T> union Pack16 {
    uint4 u;
    T e[16 / sizeof(T)];
};

__device__ __forceinline__ bool aligned16(const void *p) { return (((uintptr_t)p) & 15) == 0; }

// The transfer loops below keep many 16-byte loads in flight per thread (8 for copies, p x 2 for reductions): a peer
// load over NVLink takes a few microseconds, so bandwidth is bytes-in-flight / latency (about 2 MB per GPU at 750 GB/s).

// d (and d2) = a
__device__ __forceinline__ void copy_range(const uint8_t *a, uint8_t *d, uint8_t *d2, uint64_t bytes, int es)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    if (aligned16(a) && aligned16(d) && (!d2 || aligned16(d2))) {
        uint64_t nvec = bytes >> 4;
        const uint4 *va = (const uint4 *)a;
        uint4 *vd = (uint4 *)d, *vd2 = (uint4 *)d2;
        uint64_t i = tid;
        constexpr int U = 8;
        for (; i + (uint64_t)(U - 1) * nt < nvec; i += (uint64_t)U * nt) {
            uint4 v[U];
#pragma unroll
            for (int k = 0; k < U; ++k) v[k] = ld_stream(va + i + (uint64_t)k * nt);
#pragma unroll
            for (int k = 0; k < U; ++k) vd[i + (uint64_t)k * nt] = v[k];
            if (vd2) {
#pragma unroll
                for (int k = 0; k < U; ++k) vd2[i + (uint64_t)k * nt] = v[k];
            }
        }
        for (; i < nvec; i += nt) {
            uint4 v = ld_stream(va + i);
            vd[i] = v;
            if (vd2) vd2[i] = v;
        }
        for (uint64_t b = (nvec << 4) + tid; b < bytes; b += nt) {
            uint8_t v = a[b];
            d[b] = v;
            if (d2) d2[b] = v;
        }
    } else if (es >= 4 && ((((uintptr_t)a) | ((uintptr_t)d) | ((uintptr_t)d2)) & 3) == 0) {
        uint64_t n = bytes >> 2;
        for (uint64_t i = tid; i < n; i += nt) {
            uint32_t v = ((const uint32_t *)a)[i];
            ((uint32_t *)d)[i] = v;
            if (d2) ((uint32_t *)d2)[i] = v;
        }
    } else {
        for (uint64_t b = tid; b < bytes; b += nt) {
            uint8_t v = a[b];
            d[b] = v;
            if (d2) d2[b] = v;
        }
    }
}

// Up to p blocks of at most one 16-byte vector per thread each: the loads of eight blocks are in flight before the first
// store.  Not inlined: its 32 data registers stay out of the executor's main loop.
static __device__ __noinline__ void gather_small_blocks(const uint8_t *const *src, uint8_t *const *dst, const uint64_t *bytes, int p)
{
    const uint64_t mine = (uint64_t)threadIdx.x * 16;
    for (int i0 = 0; i0 < p; i0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (i0 + k < p && mine < bytes[i0 + k]) v[k] = ld_stream((const uint4 *)src[i0 + k] + threadIdx.x);
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (i0 + k < p && mine < bytes[i0 + k]) ((uint4 *)dst[i0 + k])[threadIdx.x] = v[k];
    }
}

// multicast store of a local range: d_mc = a on every rank
__device__ __forceinline__ void copy_range_mc(const uint8_t *a, uint8_t *d_mc, uint64_t bytes)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    uint64_t nvec = bytes >> 4;
    const uint4 *va = (const uint4 *)a;
    uint64_t i = tid;
    constexpr int U = 4;
    for (; i + (uint64_t)(U - 1) * nt < nvec; i += (uint64_t)U * nt) {
        uint4 v[U];
#pragma unroll
        for (int k = 0; k < U; ++k) v[k] = ld_stream(va + i + (uint64_t)k * nt);
#pragma unroll
        for (int k = 0; k < U; ++k) multimem_st_v4(d_mc + ((i + (uint64_t)k * nt) << 4), v[k]);
    }
    for (; i < nvec; i += nt) multimem_st_v4(d_mc + (i << 4), ld_stream(va + i));
    // the selector only picks multicast algorithms for byte counts that are multiples of 16
}

template <class T, int OP>
__device__ __forceinline__ void reduce2_range(const uint8_t *a, const uint8_t *b, uint8_t *d, uint8_t *d2, uint64_t n)
{
    using N = DNum<T>;
    const int tid = threadIdx.x, nt = blockDim.x;
    constexpr int E = 16 / sizeof(T);
    uint64_t done = 0;
    if (aligned16(a) && aligned16(b) && aligned16(d) && (!d2 || aligned16(d2))) {
        uint64_t nvec = n / E;
        constexpr int U = 4;
        uint64_t i = tid;
        for (; i + (uint64_t)(U - 1) * nt < nvec; i += (uint64_t)U * nt) {
            Pack16<T> x[U], y[U];
#pragma unroll
            for (int k = 0; k < U; ++k) {
                x[k].u = ld_stream((const uint4 *)a + i + (uint64_t)k * nt);
                y[k].u = ld_stream((const uint4 *)b + i + (uint64_t)k * nt);
            }
#pragma unroll
            for (int k = 0; k < U; ++k) {
                Pack16<T> z;
#pragma unroll
                for (int e = 0; e < E; ++e) z.e[e] = N::down(red_op<OP>(N::up(x[k].e[e]), N::up(y[k].e[e])));
                ((uint4 *)d)[i + (uint64_t)k * nt] = z.u;
                if (d2) ((uint4 *)d2)[i + (uint64_t)k * nt] = z.u;
            }
        }
        for (; i < nvec; i += nt) {
            Pack16<T> x, y, z;
            x.u = ld_stream((const uint4 *)a + i);
            y.u = ld_stream((const uint4 *)b + i);
#pragma unroll
            for (int k = 0; k < E; ++k) z.e[k] = N::down(red_op<OP>(N::up(x.e[k]), N::up(y.e[k])));
            ((uint4 *)d)[i] = z.u;
            if (d2) ((uint4 *)d2)[i] = z.u;
        }
        done = nvec * E;
    }
    const T *pa = (const T *)a, *pb = (const T *)b;
    T *pd = (T *)d, *pd2 = (T *)d2;
    for (uint64_t i = done + tid; i < n; i += nt) {
        T v = N::down(red_op<OP>(N::up(pa[i]), N::up(pb[i])));
        pd[i] = v;
        if (pd2) pd2[i] = v;
    }
}

// d (and d2) = reduction over the p sources in rank order (fixed order: bit-reproducible)
template <class T, int OP>
__device__ __forceinline__ void reduce_all_range(const uint8_t *const *src, int p, uint8_t *d, uint8_t *d2, uint64_t n)
{
    using N = DNum<T>;
    using Acc = typename N::Acc;
    const int tid = threadIdx.x, nt = blockDim.x;
    constexpr int E = 16 / sizeof(T);
    bool al = aligned16(d) && (!d2 || aligned16(d2));
    for (int q = 0; q < p; ++q) al = al && aligned16(src[q]);
    uint64_t done = 0;
    if (al) {
        uint64_t nvec = n / E;
        constexpr int B = 8;  // up to eight peers per batch, two vectors per thread: 16 loads in flight
        const uint4 *s0 = (const uint4 *)src[0], *s1 = (const uint4 *)src[p > 1 ? 1 : 0], *s2 = (const uint4 *)src[p > 2 ? 2 : 0],
                    *s3 = (const uint4 *)src[p > 3 ? 3 : 0], *s4 = (const uint4 *)src[p > 4 ? 4 : 0], *s5 = (const uint4 *)src[p > 5 ? 5 : 0],
                    *s6 = (const uint4 *)src[p > 6 ? 6 : 0], *s7 = (const uint4 *)src[p > 7 ? 7 : 0];
        for (uint64_t i = tid; i < nvec; i += 2ull * nt) {
            const uint64_t j = i + nt;
            const bool two = j < nvec;
            uint4 a0, a1, a2, a3, a4, a5, a6, a7, b0, b1, b2, b3, b4, b5, b6, b7;
            a0 = ld_stream(s0 + i);
            if (p > 1) a1 = ld_stream(s1 + i);
            if (p > 2) a2 = ld_stream(s2 + i);
            if (p > 3) a3 = ld_stream(s3 + i);
            if (p > 4) a4 = ld_stream(s4 + i);
            if (p > 5) a5 = ld_stream(s5 + i);
            if (p > 6) a6 = ld_stream(s6 + i);
            if (p > 7) a7 = ld_stream(s7 + i);
            if (two) {
                b0 = ld_stream(s0 + j);
                if (p > 1) b1 = ld_stream(s1 + j);
                if (p > 2) b2 = ld_stream(s2 + j);
                if (p > 3) b3 = ld_stream(s3 + j);
                if (p > 4) b4 = ld_stream(s4 + j);
                if (p > 5) b5 = ld_stream(s5 + j);
                if (p > 6) b6 = ld_stream(s6 + j);
                if (p > 7) b7 = ld_stream(s7 + j);
            }
            auto fold = [&](uint64_t idx, uint4 v0, uint4 v1, uint4 v2, uint4 v3, uint4 v4, uint4 v5, uint4 v6, uint4 v7) {
                Acc acc[E];
                Pack16<T> t;
                t.u = v0;
#pragma unroll
                for (int k = 0; k < E; ++k) acc[k] = N::up(t.e[k]);
                auto add = [&](uint4 v) {
                    Pack16<T> y;
                    y.u = v;
#pragma unroll
                    for (int k = 0; k < E; ++k) acc[k] = red_op<OP>(acc[k], N::up(y.e[k]));
                };
                if (p > 1) add(v1);
                if (p > 2) add(v2);
                if (p > 3) add(v3);
                if (p > 4) add(v4);
                if (p > 5) add(v5);
                if (p > 6) add(v6);
                if (p > 7) add(v7);
                for (int q = B; q < p; ++q) add(ld_stream((const uint4 *)src[q] + idx));  // more than eight ranks
                Pack16<T> z;
#pragma unroll
                for (int k = 0; k < E; ++k) z.e[k] = N::down(acc[k]);
                ((uint4 *)d)[idx] = z.u;
                if (d2) ((uint4 *)d2)[idx] = z.u;
            };
            fold(i, a0, a1, a2, a3, a4, a5, a6, a7);
            if (two) fold(j, b0, b1, b2, b3, b4, b5, b6, b7);
        }
        done = nvec * E;
    }
    T *pd = (T *)d, *pd2 = (T *)d2;
    for (uint64_t i = done + tid; i < n; i += nt) {
        Acc acc = N::up(((const T *)src[0])[i]);
        for (int q = 1; q < p; ++q) acc = red_op<OP>(acc, N::up(((const T *)src[q])[i]));
        T v = N::down(acc);
        pd[i] = v;
        if (pd2) pd2[i] = v;
    }
}

// In-switch reduction: d (unicast or multicast) and d2 = multimem.ld_reduce(mc).  `bytes` is a multiple of 16.
template <class T, int OP>
__device__ __forceinline__ void mc_reduce_range(const uint8_t *mc, uint8_t *d, bool d_is_mc, uint8_t *d2, uint64_t bytes)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    uint64_t nvec = bytes >> 4;
    constexpr int U = 8;
    uint64_t i = tid;
    for (; i + (uint64_t)(U - 1) * nt < nvec; i += (uint64_t)U * nt) {
        uint4 v[U];
#pragma unroll
        for (int k = 0; k < U; ++k) v[k] = multimem_ld_reduce<T, OP>(mc + ((i + (uint64_t)k * nt) << 4));
#pragma unroll
        for (int k = 0; k < U; ++k) {
            uint64_t idx = i + (uint64_t)k * nt;
            if (d_is_mc) multimem_st_v4(d + (idx << 4), v[k]);
            else ((uint4 *)d)[idx] = v[k];
            if (d2) ((uint4 *)d2)[idx] = v[k];
        }
    }
    for (; i < nvec; i += nt) {
        uint4 v = multimem_ld_reduce<T, OP>(mc + (i << 4));
        if (d_is_mc) multimem_st_v4(d + (i << 4), v);
        else ((uint4 *)d)[i] = v;
        if (d2) ((uint4 *)d2)[i] = v;
    }
}


// (type, operator) pairs that multimem.ld_reduce implements
template <class T, int OP> struct McSupported : std::false_type {};
template <> struct McSupported<float, HCCL_REDUCE_SUM> : std::true_type {};
#define HCCLB_MC_OK(T) \
    template <> struct McSupported<T, HCCL_REDUCE_SUM> : std::true_type {}; \
    template <> struct McSupported<T, HCCL_REDUCE_MAX> : std::true_type {}; \
    template <> struct McSupported<T, HCCL_REDUCE_MIN> : std::true_type {};
HCCLB_MC_OK(__half)
HCCLB_MC_OK(__nv_bfloat16)
HCCLB_MC_OK(int32_t)
HCCLB_MC_OK(uint32_t)
#undef HCCLB_MC_OK

// ---------------------------------------------------------------------------------------------- kernel
template <class T, int OP>
__global__ void __launch_bounds__(kExecThreads, 1) exec_plan_kernel(const RankCtx *ctxs, const ExecArgsArray args)
{
    const ExecArgs &a = args.a[blockIdx.y];
    const int chan = blockIdx.x, tid = threadIdx.x;
    // the rank context and the first steps are staged in shared memory: one coalesced read instead of a dependent
    // global load per field and step
    __shared__ RankCtx s_ctx;
    __shared__ Step s_steps[kSmemSteps];
    {
        const uint64_t *gs = (const uint64_t *)&ctxs[blockIdx.y];
        for (int i = tid; i < (int)(sizeof(RankCtx) / 8); i += blockDim.x) ((uint64_t *)&s_ctx)[i] = gs[i];
        const int nsm = a.nsteps < kSmemSteps ? a.nsteps : kSmemSteps;
        const uint64_t *gp = (const uint64_t *)a.steps;
        for (int i = tid; i < nsm * (int)(sizeof(Step) / 8); i += blockDim.x) ((uint64_t *)s_steps)[i] = gp[i];
    }
    const RankCtx &c = s_ctx;
    const int es = dtype_size(a.dtype);
    __shared__ int s_fail;
    __shared__ const uint8_t *s_src[kMaxRanks];
    __shared__ const uint8_t *s_gsrc[kMaxRanks];  // ST_GATHER_ALL: source, destination and bytes of every block of this channel
    __shared__ uint8_t *s_gdst[kMaxRanks];
    __shared__ uint64_t s_gbytes[kMaxRanks];
    if (tid == 0) s_fail = 0;
    __syncthreads();
    const int me = c.rank, p = c.nranks;
    WaitCtx w;
    w.deadline = global_timer_ns() + c.timeout_ns;
    w.abort = c.abort;
    w.local_fail = c.exit_counter + 1;
    const uint64_t half_off = a.track_done ? (a.seq & 1) * c.stage_half : 0;

    if (c.trace && tid == 0) {
        if (chan == 0) c.trace[kTraceWords - 2] = c.trace[kTraceWords - 1];  // end of the previous launch
        atomicMin((unsigned long long *)&c.trace[0], (unsigned long long)global_timer_ns());
    }
    if (a.track_done) {
        if (a.seq >= 2) {  // the peers must have left the op that used this staging half before
            if (tid < p && tid != me) {
                uint64_t seen;
                int rc = wait_flag_ge(c.flags[me] + done_index(tid), a.seq - 2, w, seen);
                if (rc) { report_failure(c, a.seq, rc, -1, tid, chan, a.seq - 2, seen); s_fail = rc; }
            }
            __syncthreads();
        }
    }
    for (int si = 0; si < a.nsteps && !s_fail; ++si) {
        const Step &s = si < kSmemSteps ? s_steps[si] : a.steps[si];
        if (chan < s.chan_lo || chan >= s.chan_lo + s.chan_n) continue;
        const int ci = chan - s.chan_lo;
        const bool tr = c.trace && tid == 0 && si < kTraceSteps;  // slowest channel of the step: atomicMax over its channels
        // ---- wait
        if (s.wait_rank != RANK_NONE) {
            const uint64_t want = flag_value(a, s, s.wait_val);
            const int nq = s.wait_rank == RANK_ALL ? p : 1;
            const int c0 = (s.flags & SF_WAIT_ALLCH) ? s.wait_clo : chan;
            const int nc = (s.flags & SF_WAIT_ALLCH) ? s.wait_cn : 1;
            for (int t = tid; t < nq * nc; t += blockDim.x) {
                int q = s.wait_rank == RANK_ALL ? t / nc : s.wait_rank;
                int cc = c0 + t % nc;
                if (q == me && !(s.flags & SF_INCLUDE_SELF)) continue;
                uint64_t seen;
                int rc = wait_flag_ge(c.flags[me] + flag_index(s.wait_bank, q, cc), want, w, seen);
                if (rc) { report_failure(c, a.seq, rc, si, q, cc, want, seen); s_fail = rc; }
            }
            __syncthreads();
            if (s_fail) break;
        }
        if (tr) atomicMax((unsigned long long *)&c.trace[1 + 3 * si], (unsigned long long)global_timer_ns());
        // ---- move / reduce
        uint64_t lo, hi;
        switch (s.op) {
            case ST_COPY: {
                chan_range(s.count, es, s.chan_n, ci, lo, hi);
                if (hi > lo) {
                    const uint8_t *src = resolve_addr(c, a, s.a_buf, s.a_rank, s.a_off, half_off) + lo * es;
                    uint8_t *dst = resolve_addr(c, a, s.d_buf, s.d_rank, s.d_off, half_off) + lo * es;
                    if (s.d_rank == RANK_ALL) copy_range_mc(src, dst, (hi - lo) * es);
                    else {
                        uint8_t *d2 = s.d2_buf != BUF_NONE ? resolve_addr(c, a, s.d2_buf, RANK_SELF, s.d2_off, half_off) + lo * es : nullptr;
                        copy_range(src, dst, d2, (hi - lo) * es, es);
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
                    reduce2_range<T, OP>(pa, pb, pd, pd2, hi - lo);
                }
                break;
            }
            case ST_REDUCE_ALL: {
                chan_range(s.count, es, s.chan_n, ci, lo, hi);
                if (hi > lo) {
                    if (tid < p) s_src[tid] = resolve_addr(c, a, s.a_buf, tid, s.a_off, half_off) + lo * es;
                    __syncthreads();
                    uint8_t *pd = resolve_addr(c, a, s.d_buf, s.d_rank, s.d_off, half_off) + lo * es;
                    uint8_t *pd2 = s.d2_buf != BUF_NONE ? resolve_addr(c, a, s.d2_buf, RANK_SELF, s.d2_off, half_off) + lo * es : nullptr;
                    reduce_all_range<T, OP>(s_src, p, pd, pd2, hi - lo);
                }
                break;
            }
            case ST_MC_REDUCE: {
                chan_range(s.count, es, s.chan_n, ci, lo, hi);
                if (hi > lo) {
                    const uint8_t *mc = resolve_addr(c, a, s.a_buf, RANK_ALL, s.a_off, half_off) + lo * es;
                    uint8_t *pd = resolve_addr(c, a, s.d_buf, s.d_rank, s.d_off, half_off) + lo * es;
                    uint8_t *pd2 = s.d2_buf != BUF_NONE ? resolve_addr(c, a, s.d2_buf, RANK_SELF, s.d2_off, half_off) + lo * es : nullptr;
                    if constexpr (McSupported<T, OP>::value) mc_reduce_range<T, OP>(mc, pd, s.d_rank == RANK_ALL, pd2, (hi - lo) * es);
                }
                break;
            }
            case ST_GATHER_ALL: {
                // Small blocks (at most one 16-byte vector per thread and block): the loads of all blocks are issued before
                // the first store, so the step costs one memory round trip instead of one per block (p NVLink latencies in
                // the gather phase of a two-shot AllReduce of a few MiB).  Threads tid < p describe the blocks.
                if (tid < p) {
                    const int q = (me + tid) % p;
                    uint64_t cnt = s.count;
                    if (s.limit) {
                        uint64_t start = (uint64_t)q * s.count;
                        cnt = start >= s.limit ? 0 : (s.limit - start < s.count ? s.limit - start : s.count);
                    }
                    if (q == me && (s.flags & SF_SKIP_SELF)) cnt = 0;
                    chan_range(cnt, es, s.chan_n, ci, lo, hi);
                    const int src_rank = s.a_rank == RANK_ALL ? q : RANK_SELF;
                    s_gsrc[tid] = resolve_addr(c, a, s.a_buf, src_rank, s.a_off + (uint64_t)q * s.a_stride, half_off) + lo * es;
                    s_gdst[tid] = resolve_addr(c, a, s.d_buf, RANK_SELF, s.d_off + (uint64_t)q * s.d_stride, half_off) + lo * es;
                    s_gbytes[tid] = hi > lo ? (hi - lo) * es : 0;
                }
                __syncthreads();
                bool small = true;
                for (int i = 0; i < p; ++i)
                    small = small && s_gbytes[i] <= (uint64_t)16 * blockDim.x && (s_gbytes[i] & 15) == 0 && aligned16(s_gsrc[i]) && aligned16(s_gdst[i]);
                if (small) {
                    gather_small_blocks(s_gsrc, s_gdst, s_gbytes, p);
                } else {
                    for (int i = 0; i < p; ++i)
                        if (s_gbytes[i]) copy_range(s_gsrc[i], s_gdst[i], nullptr, s_gbytes[i], es);
                }
                __syncthreads();  // the block descriptions are rewritten by the next gather step
                break;
            }
            default: break;
        }
        if (c.trace && si < kTraceSteps) {  // uniform across the CTA
            __syncthreads();
            if (tid == 0) atomicMax((unsigned long long *)&c.trace[2 + 3 * si], (unsigned long long)global_timer_ns());
        }
        // ---- signal
        if (s.sig_rank != RANK_NONE) {
            __syncthreads();  // every thread's stores of this step precede the release (a system-scope fence in itself) of the signalling threads
            const uint64_t val = flag_value(a, s, s.sig_val);
            if (s.sig_rank == RANK_ALL) {
                if (tid < p && (tid != me || (s.flags & SF_INCLUDE_SELF))) { st_release_sys(c.flags[tid] + flag_index(s.sig_bank, me, chan), val); }
            } else if (tid == 0 && (s.sig_rank != me || (s.flags & SF_INCLUDE_SELF))) {
                st_release_sys(c.flags[s.sig_rank] + flag_index(s.sig_bank, me, chan), val);
            }
        }
        if (tr) atomicMax((unsigned long long *)&c.trace[3 + 3 * si], (unsigned long long)global_timer_ns());
    }
    if (c.trace && tid == 0) atomicMax((unsigned long long *)&c.trace[kTraceWords - 1], (unsigned long long)global_timer_ns());
    // ---- completion: the last CTA of this rank tells every peer that this op no longer touches their memory
    if (a.track_done) {
        __syncthreads();
        __shared__ int s_last;
        if (tid == 0) {
            __threadfence();
            unsigned prev = atomicAdd(c.exit_counter, 1u);
            s_last = prev == gridDim.x - 1;
            if (s_last) *c.exit_counter = 0;
        }
        __syncthreads();
        if (s_last && !s_fail) {
            if (tid < p && tid != me) { st_release_sys(c.flags[tid] + done_index(me), a.seq); }
            if (tid == 0) *c.dev_tail = a.seq;  // read by the heartbeat thread with an asynchronous copy
        }
    }
}


// Defines exec_kernel_<name>(op): the kernel entry for element type T and reduction `op`.
#define HCCLB_INSTANTIATE_EXEC(T, name)                                                          \
    const void *exec_kernel_##name(int op)                                                       \
    {                                                                                            \
        switch (op) {                                                                            \
            case HCCL_REDUCE_SUM: return (const void *)exec_plan_kernel<T, HCCL_REDUCE_SUM>;     \
            case HCCL_REDUCE_PROD: return (const void *)exec_plan_kernel<T, HCCL_REDUCE_PROD>;   \
            case HCCL_REDUCE_MAX: return (const void *)exec_plan_kernel<T, HCCL_REDUCE_MAX>;     \
            default: return (const void *)exec_plan_kernel<T, HCCL_REDUCE_MIN>;                  \
        }                                                                                        \
    }

}  // namespace hcclb
