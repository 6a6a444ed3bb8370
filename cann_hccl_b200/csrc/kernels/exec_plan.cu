// Device plan executor for sm_100a: one CTA per channel interprets the step list of its rank.  Peers' staging
// buffers are read and written directly over NVLink through their peer mappings (ld/st.global) or through the NVLS
// multicast mapping (multimem.ld_reduce / multimem.st); the reduction operator is applied in registers while the
// data moves, so no separate elementwise kernel and no library collective runs.  Flags are 64-bit words in the
// peers' flag pages, written with st.release.sys and polled with ld.acquire.sys; every poll loop is bounded by
// the communicator's timeout and by the abort word, after which the CTA records a status block and returns.
//
// This kernel replaces the reference's AIV kernel family (algorithm/base/alg_aiv_template/*.h: CpGM2GM,
// SetFlagNew / CheckFlagNew in aiv_communication_base.h:408-575) and the SDMA/notify task lists of the
// host-orchestrated path; unlike CheckFlagNew its waits cannot spin forever.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "algo/plan.h"
#include "algo/resolve.h"
#include "common/log.h"
#include "kernels/prims.cuh"

namespace hcclb {

constexpr int kExecThreads = 512;

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

// d (and d2) = a
__device__ void copy_range(const uint8_t *a, uint8_t *d, uint8_t *d2, uint64_t bytes, int es)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    if (aligned16(a) && aligned16(d) && (!d2 || aligned16(d2))) {
        uint64_t nvec = bytes >> 4;
        const uint4 *va = (const uint4 *)a;
        uint4 *vd = (uint4 *)d, *vd2 = (uint4 *)d2;
        uint64_t i = tid;
        for (; i + 3ull * nt < nvec; i += 4ull * nt) {
            uint4 v0 = ld_stream(va + i), v1 = ld_stream(va + i + nt), v2 = ld_stream(va + i + 2 * nt), v3 = ld_stream(va + i + 3 * nt);
            vd[i] = v0; vd[i + nt] = v1; vd[i + 2 * nt] = v2; vd[i + 3 * nt] = v3;
            if (vd2) { vd2[i] = v0; vd2[i + nt] = v1; vd2[i + 2 * nt] = v2; vd2[i + 3 * nt] = v3; }
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

// multicast store of a local range: d_mc = a on every rank
__device__ void copy_range_mc(const uint8_t *a, uint8_t *d_mc, uint64_t bytes)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    uint64_t nvec = bytes >> 4;
    const uint4 *va = (const uint4 *)a;
    for (uint64_t i = tid; i < nvec; i += nt) multimem_st_v4(d_mc + (i << 4), ld_stream(va + i));
    // the selector only picks multicast algorithms for byte counts that are multiples of 16
}

template <class T, int OP>
__device__ void reduce2_range(const uint8_t *a, const uint8_t *b, uint8_t *d, uint8_t *d2, uint64_t n)
{
    using N = DNum<T>;
    const int tid = threadIdx.x, nt = blockDim.x;
    constexpr int E = 16 / sizeof(T);
    uint64_t done = 0;
    if (aligned16(a) && aligned16(b) && aligned16(d) && (!d2 || aligned16(d2))) {
        uint64_t nvec = n / E;
        for (uint64_t i = tid; i < nvec; i += nt) {
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

// d (and d2) = reduction over the p sources in rank order
template <class T, int OP>
__device__ void reduce_all_range(const uint8_t *const *src, int p, uint8_t *d, uint8_t *d2, uint64_t n)
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
        for (uint64_t i = tid; i < nvec; i += nt) {
            Acc acc[E];
            Pack16<T> x;
            x.u = ld_stream((const uint4 *)src[0] + i);
#pragma unroll
            for (int k = 0; k < E; ++k) acc[k] = N::up(x.e[k]);
            int q = 1;
            for (; q + 3 < p; q += 4) {  // four peers' loads in flight together
                Pack16<T> y0, y1, y2, y3;
                y0.u = ld_stream((const uint4 *)src[q] + i);
                y1.u = ld_stream((const uint4 *)src[q + 1] + i);
                y2.u = ld_stream((const uint4 *)src[q + 2] + i);
                y3.u = ld_stream((const uint4 *)src[q + 3] + i);
#pragma unroll
                for (int k = 0; k < E; ++k) {
                    acc[k] = red_op<OP>(acc[k], N::up(y0.e[k]));
                    acc[k] = red_op<OP>(acc[k], N::up(y1.e[k]));
                    acc[k] = red_op<OP>(acc[k], N::up(y2.e[k]));
                    acc[k] = red_op<OP>(acc[k], N::up(y3.e[k]));
                }
            }
            for (; q < p; ++q) {
                Pack16<T> y;
                y.u = ld_stream((const uint4 *)src[q] + i);
#pragma unroll
                for (int k = 0; k < E; ++k) acc[k] = red_op<OP>(acc[k], N::up(y.e[k]));
            }
            Pack16<T> z;
#pragma unroll
            for (int k = 0; k < E; ++k) z.e[k] = N::down(acc[k]);
            ((uint4 *)d)[i] = z.u;
            if (d2) ((uint4 *)d2)[i] = z.u;
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
__device__ void mc_reduce_range(const uint8_t *mc, uint8_t *d, bool d_is_mc, uint8_t *d2, uint64_t bytes)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    uint64_t nvec = bytes >> 4;
    for (uint64_t i = tid; i < nvec; i += nt) {
        uint4 v = multimem_ld_reduce<T, OP>(mc + (i << 4));
        if (d_is_mc) multimem_st_v4(d + (i << 4), v);
        else ((uint4 *)d)[i] = v;
        if (d2) ((uint4 *)d2)[i] = v;
    }
}

#define HCCLB_DISPATCH_OP(FN, T, op, ...)                                   \
    switch (op) {                                                           \
        case HCCL_REDUCE_SUM: FN<T, HCCL_REDUCE_SUM>(__VA_ARGS__); break;   \
        case HCCL_REDUCE_PROD: FN<T, HCCL_REDUCE_PROD>(__VA_ARGS__); break; \
        case HCCL_REDUCE_MAX: FN<T, HCCL_REDUCE_MAX>(__VA_ARGS__); break;   \
        default: FN<T, HCCL_REDUCE_MIN>(__VA_ARGS__); break;                \
    }
#define HCCLB_DISPATCH(FN, dtype, op, ...)                                                        \
    switch (dtype) {                                                                              \
        case HCCL_DATA_TYPE_INT8: HCCLB_DISPATCH_OP(FN, int8_t, op, __VA_ARGS__) break;           \
        case HCCL_DATA_TYPE_UINT8: HCCLB_DISPATCH_OP(FN, uint8_t, op, __VA_ARGS__) break;         \
        case HCCL_DATA_TYPE_INT16: HCCLB_DISPATCH_OP(FN, int16_t, op, __VA_ARGS__) break;         \
        case HCCL_DATA_TYPE_UINT16: HCCLB_DISPATCH_OP(FN, uint16_t, op, __VA_ARGS__) break;       \
        case HCCL_DATA_TYPE_INT32: HCCLB_DISPATCH_OP(FN, int32_t, op, __VA_ARGS__) break;         \
        case HCCL_DATA_TYPE_UINT32: HCCLB_DISPATCH_OP(FN, uint32_t, op, __VA_ARGS__) break;       \
        case HCCL_DATA_TYPE_INT64: HCCLB_DISPATCH_OP(FN, long long, op, __VA_ARGS__) break;       \
        case HCCL_DATA_TYPE_UINT64: HCCLB_DISPATCH_OP(FN, unsigned long long, op, __VA_ARGS__) break; \
        case HCCL_DATA_TYPE_FP32: HCCLB_DISPATCH_OP(FN, float, op, __VA_ARGS__) break;            \
        case HCCL_DATA_TYPE_FP64: HCCLB_DISPATCH_OP(FN, double, op, __VA_ARGS__) break;           \
        case HCCL_DATA_TYPE_FP16: HCCLB_DISPATCH_OP(FN, __half, op, __VA_ARGS__) break;           \
        case HCCL_DATA_TYPE_BFP16: HCCLB_DISPATCH_OP(FN, __nv_bfloat16, op, __VA_ARGS__) break;   \
        default: break;                                                                           \
    }

// multimem.ld_reduce exists for a subset of (type, op); the selector never sends anything else here
__device__ void mc_reduce_dispatch(int dtype, int op, const uint8_t *mc, uint8_t *d, bool d_is_mc, uint8_t *d2, uint64_t bytes)
{
    switch (dtype) {
        case HCCL_DATA_TYPE_FP32: mc_reduce_range<float, HCCL_REDUCE_SUM>(mc, d, d_is_mc, d2, bytes); break;
        case HCCL_DATA_TYPE_FP16:
            if (op == HCCL_REDUCE_SUM) mc_reduce_range<__half, HCCL_REDUCE_SUM>(mc, d, d_is_mc, d2, bytes);
            else if (op == HCCL_REDUCE_MAX) mc_reduce_range<__half, HCCL_REDUCE_MAX>(mc, d, d_is_mc, d2, bytes);
            else mc_reduce_range<__half, HCCL_REDUCE_MIN>(mc, d, d_is_mc, d2, bytes);
            break;
        case HCCL_DATA_TYPE_BFP16:
            if (op == HCCL_REDUCE_SUM) mc_reduce_range<__nv_bfloat16, HCCL_REDUCE_SUM>(mc, d, d_is_mc, d2, bytes);
            else if (op == HCCL_REDUCE_MAX) mc_reduce_range<__nv_bfloat16, HCCL_REDUCE_MAX>(mc, d, d_is_mc, d2, bytes);
            else mc_reduce_range<__nv_bfloat16, HCCL_REDUCE_MIN>(mc, d, d_is_mc, d2, bytes);
            break;
        case HCCL_DATA_TYPE_INT32:
            if (op == HCCL_REDUCE_SUM) mc_reduce_range<int32_t, HCCL_REDUCE_SUM>(mc, d, d_is_mc, d2, bytes);
            else if (op == HCCL_REDUCE_MAX) mc_reduce_range<int32_t, HCCL_REDUCE_MAX>(mc, d, d_is_mc, d2, bytes);
            else mc_reduce_range<int32_t, HCCL_REDUCE_MIN>(mc, d, d_is_mc, d2, bytes);
            break;
        case HCCL_DATA_TYPE_UINT32:
            if (op == HCCL_REDUCE_SUM) mc_reduce_range<uint32_t, HCCL_REDUCE_SUM>(mc, d, d_is_mc, d2, bytes);
            else if (op == HCCL_REDUCE_MAX) mc_reduce_range<uint32_t, HCCL_REDUCE_MAX>(mc, d, d_is_mc, d2, bytes);
            else mc_reduce_range<uint32_t, HCCL_REDUCE_MIN>(mc, d, d_is_mc, d2, bytes);
            break;
        default: break;
    }
}

// ---------------------------------------------------------------------------------------------- kernel
__global__ void __launch_bounds__(kExecThreads, 1) exec_plan_kernel(const RankCtx *ctxs, const ExecArgsArray args)
{
    const RankCtx &c = ctxs[blockIdx.y];
    const ExecArgs &a = args.a[blockIdx.y];
    const int chan = blockIdx.x, tid = threadIdx.x, me = c.rank, p = c.nranks;
    const int es = dtype_size(a.dtype);
    __shared__ int s_fail;
    __shared__ const uint8_t *s_src[kMaxRanks];
    if (tid == 0) s_fail = 0;
    __syncthreads();
    WaitCtx w;
    w.deadline = global_timer_ns() + c.timeout_ns;
    w.abort = c.abort;
    w.local_fail = c.exit_counter + 1;
    const uint64_t half_off = a.track_done ? (a.seq & 1) * c.stage_half : 0;

    if (a.track_done) {
        if (chan == 0 && tid == 0) *(volatile uint64_t *)&c.status->head = a.seq;
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
        const Step &s = a.steps[si];
        if (chan < s.chan_lo || chan >= s.chan_lo + s.chan_n) continue;
        const int ci = chan - s.chan_lo;
        // ---- wait
        if (s.wait_rank != RANK_NONE) {
            const uint64_t want = flag_value(a, s, s.wait_val);
            const int nq = s.wait_rank == RANK_ALL ? p : 1;
            const int c0 = (s.flags & SF_WAIT_ALLCH) ? s.wait_clo : chan;
            const int nc = (s.flags & SF_WAIT_ALLCH) ? s.wait_cn : 1;
            for (int t = tid; t < nq * nc; t += blockDim.x) {
                int q = s.wait_rank == RANK_ALL ? t / nc : s.wait_rank;
                int cc = c0 + t % nc;
                if (q == me) continue;
                uint64_t seen;
                int rc = wait_flag_ge(c.flags[me] + flag_index(s.wait_bank, q, cc), want, w, seen);
                if (rc) { report_failure(c, a.seq, rc, si, q, cc, want, seen); s_fail = rc; }
            }
            __syncthreads();
            if (s_fail) break;
        }
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
                    HCCLB_DISPATCH(reduce2_range, a.dtype, a.redop, pa, pb, pd, pd2, hi - lo)
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
                    HCCLB_DISPATCH(reduce_all_range, a.dtype, a.redop, s_src, p, pd, pd2, hi - lo)
                }
                break;
            }
            case ST_MC_REDUCE: {
                chan_range(s.count, es, s.chan_n, ci, lo, hi);
                if (hi > lo) {
                    const uint8_t *mc = resolve_addr(c, a, s.a_buf, RANK_ALL, s.a_off, half_off) + lo * es;
                    uint8_t *pd = resolve_addr(c, a, s.d_buf, s.d_rank, s.d_off, half_off) + lo * es;
                    uint8_t *pd2 = s.d2_buf != BUF_NONE ? resolve_addr(c, a, s.d2_buf, RANK_SELF, s.d2_off, half_off) + lo * es : nullptr;
                    mc_reduce_dispatch(a.dtype, a.redop, mc, pd, s.d_rank == RANK_ALL, pd2, (hi - lo) * es);
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
                    copy_range(resolve_addr(c, a, s.a_buf, src_rank, s.a_off + (uint64_t)q * s.a_stride, half_off) + lo * es,
                               resolve_addr(c, a, s.d_buf, RANK_SELF, s.d_off + (uint64_t)q * s.d_stride, half_off) + lo * es, nullptr,
                               (hi - lo) * es, es);
                }
                break;
            }
            default: break;
        }
        // ---- signal
        if (s.sig_rank != RANK_NONE) {
            __syncthreads();  // every thread's stores of this step precede the fence of the signalling threads
            const uint64_t val = flag_value(a, s, s.sig_val);
            if (s.sig_rank == RANK_ALL) {
                if (tid < p && tid != me) { fence_sys(); st_release_sys(c.flags[tid] + flag_index(s.sig_bank, me, chan), val); }
            } else if (tid == 0 && s.sig_rank != me) {
                fence_sys();
                st_release_sys(c.flags[s.sig_rank] + flag_index(s.sig_bank, me, chan), val);
            }
        }
    }
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
            if (tid < p && tid != me) { fence_sys(); st_release_sys(c.flags[tid] + done_index(me), a.seq); }
            if (tid == 0) *(volatile uint64_t *)&c.status->tail = a.seq;
        }
    }
}

HcclResult launch_exec_plan(const RankCtx *dev_ctx, const ExecArgs *args, int nlocal, int nchan, void *stream)
{
    if (nlocal < 1 || nlocal > kMaxRanks || nchan < 1 || nchan > kMaxChannels) return HCCL_E_PARA;
    ExecArgsArray arr;
    for (int i = 0; i < nlocal; ++i) arr.a[i] = args[i];
    dim3 grid((unsigned)nchan, (unsigned)nlocal), block(kExecThreads);
    cudaError_t e;
    if (nlocal > 1) {
        // virtual ranks of one GPU wait on one another: all their CTAs must be resident at the same time
        void *kargs[] = {(void *)&dev_ctx, (void *)&arr};
        e = cudaLaunchCooperativeKernel((const void *)exec_plan_kernel, grid, block, kargs, 0, (cudaStream_t)stream);
    } else {
        exec_plan_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(dev_ctx, arr);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        HLOG_ERROR("executor launch failed (grid %dx%d): %s", nchan, nlocal, cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
