// Small-message AllReduce for sm_100a, low-latency protocol: every rank pushes its contribution straight into a
// mailbox on every peer as 16-byte lines {data, tag, data, tag} (8 payload bytes per line; a line is valid when both
// tags equal this operation's tag), then polls its own mailboxes and reduces in rank order.  No fence, no separate
// flag hop, no staging copy and no step table: one NVLink store latency separates the first instruction from the
// result.  This is the latency path that the reference gives to its AIV small-data kernels
// (algorithm/base/alg_aiv_template/aiv_all_reduce_910b_smalldata.h: one-shot, <= 64 KB); there the flag is a
// separate 32-byte word and the wait is unbounded, here the flag travels with the data and every poll is bounded.
//
// Two-shot form for three and more ranks and messages of a few MiB (the reference's mid-data class,
// alg_aiv_template/aiv_all_reduce_910b_middata.h): a rank pushes slice q of its input to rank q only, reduces its own slice
// from the p - 1 lines it polls, stores the result and pushes it, again as tagged lines, to every peer, and collects the
// other slices the same way.  Each byte crosses a link about 4 (p - 1) / p times instead of 2 (p - 1) times, still with no
// fence and no separate flag hop.
//
// Mailboxes are double buffered by the parity of the LL operation count: a rank can only start LL operation k+2 after
// it has received every peer's lines of k+1, which those peers sent after they finished reading k.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "common/log.h"
#include "kernels/ar_ll.h"
#include "kernels/prims.cuh"

namespace hcclb {

namespace {

template <class T> struct LNum { using Acc = T; static __device__ __forceinline__ Acc up(T v) { return v; } static __device__ __forceinline__ T down(Acc v) { return v; } };
template <> struct LNum<__half> { using Acc = float; static __device__ __forceinline__ float up(__half v) { return __half2float(v); } static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); } };
template <> struct LNum<__nv_bfloat16> { using Acc = float; static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); } static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); } };

template <int OP, class A> __device__ __forceinline__ A ll_op(A x, A y)
{
    if (OP == HCCL_REDUCE_SUM) return (A)(x + y);
    if (OP == HCCL_REDUCE_PROD) return (A)(x * y);
    if (OP == HCCL_REDUCE_MAX) return x > y ? x : y;
    return x < y ? x : y;
}

template <class T> union Pay8 {
    uint2 u;
    T e[8 / sizeof(T)];
};

__device__ __forceinline__ void st_line(uint8_t *p, uint32_t d0, uint32_t d1, uint32_t tag)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(d0), "r"(tag), "r"(d1), "r"(tag) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint8_t *p)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <class T, int OP>
__global__ void __launch_bounds__(kLlThreads) ar_ll_kernel(const LlArgsArray args)
{
    const LlArgs &a = args.a[blockIdx.y];
    using N = LNum<T>;
    using Acc = typename N::Acc;
    constexpr int E = 8 / sizeof(T);
    const int me = a.rank, p = a.nranks;
    const uint64_t nlines = (a.count + E - 1) / E;
    const uint64_t parity_off = (uint64_t)a.parity * (uint64_t)p * a.slot_bytes;
    const uint64_t deadline = global_timer_ns() + a.timeout_ns;
    const T *in = (const T *)a.in;
    T *out = (T *)a.out;
    // buffers that are only element-aligned take the element-wise path: which path a rank takes is its own business, the
    // lines on the wire are the same
    const bool in8 = ((uintptr_t)in & 7) == 0, out8 = ((uintptr_t)out & 7) == 0;
    const uint64_t first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (uint64_t)gridDim.x * blockDim.x;
    auto load_mine = [&](uint64_t line) {
        Pay8<T> mine;
        const uint64_t e0 = line * E;
        if (in8 && e0 + E <= a.count) mine.u = *(const uint2 *)(in + e0);
        else {
            mine.u = make_uint2(0, 0);
            for (int k = 0; k < E; ++k)
                if (e0 + k < a.count) mine.e[k] = in[e0 + k];
        }
        return mine;
    };
    // phase 1: push every line of this thread to every peer; the stores pipeline freely
    for (uint64_t line = first; line < nlines; line += stride) {
        Pay8<T> mine = load_mine(line);
        const uint64_t loff = parity_off + (uint64_t)me * a.slot_bytes + line * 16;
        for (int i = 1; i < p; ++i) {  // start at the next rank so that the peers' links are hit evenly
            int q = me + i;
            if (q >= p) q -= p;
            st_line(a.ll[q] + loff, mine.u.x, mine.u.y, a.tag);
        }
    }
    // phase 2: collect the peers' lines (mostly arrived by now) and reduce in rank order
    for (uint64_t line = first; line < nlines; line += stride) {
        Pay8<T> mine = load_mine(line);
        const uint64_t e0 = line * E;
        Acc acc[E];
        bool have = false;
        bool failed = false;
        for (int q = 0; q < p && !failed; ++q) {
            Pay8<T> v;
            if (q == me) v = mine;
            else {
                const uint8_t *src = a.ll[me] + parity_off + (uint64_t)q * a.slot_bytes + line * 16;
                uint4 l = ld_line(src);
                for (uint32_t it = 0; l.y != a.tag || l.w != a.tag; ++it) {
                    if ((it & 255) == 255) {
                        int code = 0;
                        if (global_timer_ns() > deadline) code = HCCL_E_TIMEOUT;
                        else if (*(volatile uint32_t *)a.local_fail) code = (int)*(volatile uint32_t *)a.local_fail;
                        else if ((it & 8191) == 8191 && *a.abort) code = *a.abort == 2 ? HCCL_E_REMOTE : HCCL_E_SUSPENDING;
                        if (code) {
                            if (atomicCAS(a.local_fail, 0u, (uint32_t)code) == 0u) {
                                DevStatus *s = a.status;
                                s->step = 0; s->peer = q; s->chan = blockIdx.x; s->expected = a.tag; s->seen = l.y; s->seq = a.seq;
                                __threadfence_system();
                                *(volatile uint32_t *)&s->code = (uint32_t)code;
                            }
                            failed = true;
                            break;
                        }
                    }
                    l = ld_line(src);
                }
                v.u = make_uint2(l.x, l.z);
            }
            if (!have) {
#pragma unroll
                for (int k = 0; k < E; ++k) acc[k] = N::up(v.e[k]);
                have = true;
            } else {
#pragma unroll
                for (int k = 0; k < E; ++k) acc[k] = ll_op<OP>(acc[k], N::up(v.e[k]));
            }
        }
        if (failed) return;  // head stays ahead of tail: the heartbeat reports the op as stuck / failed
        Pay8<T> r;
#pragma unroll
        for (int k = 0; k < E; ++k) r.e[k] = N::down(acc[k]);
        if (out8 && e0 + E <= a.count) *(uint2 *)(out + e0) = r.u;
        else
            for (int k = 0; k < E; ++k)
                if (e0 + k < a.count) out[e0 + k] = r.e[k];
    }
    // op-execution counter: the last CTA of this rank moves the tail up to the head the host set at launch
    __syncthreads();
    if (threadIdx.x == 0 && a.exit_counter) {
        __threadfence();
        if (atomicAdd(a.exit_counter, 1u) == gridDim.x - 1) {
            *a.exit_counter = 0;
            *a.dev_tail = a.exe_id;
        }
    }
}

// Polls one line until both tags match; false when the wait was given up (the first failure of the rank is recorded).
__device__ __forceinline__ bool ll_poll(const LlArgs &a, const uint8_t *src, uint64_t deadline, int peer, uint4 &l)
{
    l = ld_line(src);
    for (uint32_t it = 0; l.y != a.tag || l.w != a.tag; ++it) {
        if ((it & 255) == 255) {
            int code = 0;
            if (global_timer_ns() > deadline) code = HCCL_E_TIMEOUT;
            else if (*(volatile uint32_t *)a.local_fail) code = (int)*(volatile uint32_t *)a.local_fail;
            else if ((it & 8191) == 8191 && *a.abort) code = *a.abort == 2 ? HCCL_E_REMOTE : HCCL_E_SUSPENDING;
            if (code) {
                if (atomicCAS(a.local_fail, 0u, (uint32_t)code) == 0u) {
                    DevStatus *s = a.status;
                    s->step = 0; s->peer = peer; s->chan = blockIdx.x; s->expected = a.tag; s->seen = l.y; s->seq = a.seq;
                    __threadfence_system();
                    *(volatile uint32_t *)&s->code = (uint32_t)code;
                }
                return false;
            }
        }
        l = ld_line(src);
    }
    return true;
}

// Two-shot: the mailbox half of a parity holds area A (slices pushed to their owner, one piece per source rank) followed by
// area B (reduced slices pushed by their owner, one piece per owner); a piece is piece_bytes long.
template <class T, int OP>
__global__ void __launch_bounds__(kLlThreads) ar_ll2_kernel(const LlArgsArray args)
{
    const LlArgs &a = args.a[blockIdx.y];
    using N = LNum<T>;
    using Acc = typename N::Acc;
    constexpr int E = 8 / sizeof(T);
    const int me = a.rank, p = a.nranks;
    const uint64_t nlines = (a.count + E - 1) / E;
    const uint64_t ls = (nlines + p - 1) / p;  // lines per slice
    const uint64_t half = (uint64_t)p * a.slot_bytes, piece = half / 2 / p;
    const uint64_t base_a = (uint64_t)a.parity * half, base_b = base_a + half / 2;
    const uint64_t deadline = global_timer_ns() + a.timeout_ns;
    const T *in = (const T *)a.in;
    T *out = (T *)a.out;
    // buffers that are only element-aligned take the element-wise path: which path a rank takes is its own business, the
    // lines on the wire are the same
    const bool in8 = ((uintptr_t)in & 7) == 0, out8 = ((uintptr_t)out & 7) == 0;
    const uint64_t first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (uint64_t)gridDim.x * blockDim.x;
    auto load_mine = [&](uint64_t line) {
        Pay8<T> mine;
        const uint64_t e0 = line * E;
        if (in8 && e0 + E <= a.count) mine.u = *(const uint2 *)(in + e0);
        else {
            mine.u = make_uint2(0, 0);
            for (int k = 0; k < E; ++k)
                if (e0 + k < a.count) mine.e[k] = in[e0 + k];
        }
        return mine;
    };
    auto store_out = [&](uint64_t line, Pay8<T> r) {
        const uint64_t e0 = line * E;
        if (out8 && e0 + E <= a.count) *(uint2 *)(out + e0) = r.u;
        else
            for (int k = 0; k < E; ++k)
                if (e0 + k < a.count) out[e0 + k] = r.e[k];
    };
    const uint64_t my_lo = ls * me < nlines ? ls * me : nlines, my_hi = my_lo + ls < nlines ? my_lo + ls : nlines;
    // phase 1: every line outside my slice goes to its owner's area A, piece `me`
    for (uint64_t line = first; line < nlines; line += stride) {
        const int q = (int)(line / ls);
        if (q == me) continue;
        Pay8<T> mine = load_mine(line);
        st_line(a.ll[q] + base_a + (uint64_t)me * piece + (line - (uint64_t)q * ls) * 16, mine.u.x, mine.u.y, a.tag);
    }
    // phase 2: reduce my slice in rank order, store it and push it to every peer's area B, piece `me`
    bool failed = false;
    for (uint64_t line = my_lo + first; line < my_hi && !failed; line += stride) {
        const uint64_t jj = line - my_lo;
        Pay8<T> mine = load_mine(line);
        Acc acc[E];
        for (int q = 0; q < p && !failed; ++q) {
            Pay8<T> v;
            if (q == me) v = mine;
            else {
                uint4 l;
                if (!ll_poll(a, a.ll[me] + base_a + (uint64_t)q * piece + jj * 16, deadline, q, l)) { failed = true; break; }
                v.u = make_uint2(l.x, l.z);
            }
            if (q == 0) {
#pragma unroll
                for (int k = 0; k < E; ++k) acc[k] = N::up(v.e[k]);
            } else {
#pragma unroll
                for (int k = 0; k < E; ++k) acc[k] = ll_op<OP>(acc[k], N::up(v.e[k]));
            }
        }
        if (failed) break;
        Pay8<T> r;
#pragma unroll
        for (int k = 0; k < E; ++k) r.e[k] = N::down(acc[k]);
        store_out(line, r);
        for (int i = 1; i < p; ++i) {
            int q = me + i;
            if (q >= p) q -= p;
            st_line(a.ll[q] + base_b + (uint64_t)me * piece + jj * 16, r.u.x, r.u.y, a.tag);
        }
    }
    // phase 3: the other slices arrive reduced in area B
    for (uint64_t line = first; line < nlines && !failed; line += stride) {
        const int q = (int)(line / ls);
        if (q == me) continue;
        uint4 l;
        if (!ll_poll(a, a.ll[me] + base_b + (uint64_t)q * piece + (line - (uint64_t)q * ls) * 16, deadline, q, l)) { failed = true; break; }
        Pay8<T> r;
        r.u = make_uint2(l.x, l.z);
        store_out(line, r);
    }
    if (failed) return;  // head stays ahead of tail: the heartbeat reports the op as stuck / failed
    __syncthreads();
    if (threadIdx.x == 0 && a.exit_counter) {
        __threadfence();
        if (atomicAdd(a.exit_counter, 1u) == gridDim.x - 1) {
            *a.exit_counter = 0;
            *a.dev_tail = a.exe_id;
        }
    }
}

// ReduceScatter and AllGather in the LL protocol: the two phases of the two-shot AllReduce as collectives of their own.
// a.count = elements of one rank's block.  ReduceScatter: block q of my input goes to its owner's area A (piece `me`), I
// reduce my block from the p - 1 pieces that arrive plus my own.  AllGather: my block goes to area B (piece `me`) of every
// peer, the peers' blocks arrive in mine.  Blocks start wherever the caller's count puts them, so loads and stores fall back
// to single elements where a block is not 8-byte aligned.
template <class T, int OP>
__global__ void __launch_bounds__(kLlThreads) ll_rsag_kernel(const LlArgsArray args)
{
    const LlArgs &a = args.a[blockIdx.y];
    using N = LNum<T>;
    using Acc = typename N::Acc;
    constexpr int E = 8 / sizeof(T);
    const int me = a.rank, p = a.nranks;
    const bool rs = a.two_shot == LL_REDUCE_SCATTER;
    const uint64_t bl = (a.count + E - 1) / E;  // lines per block
    const uint64_t half = (uint64_t)p * a.slot_bytes, piece = half / 2 / p;
    const uint64_t base_a = (uint64_t)a.parity * half, base_b = base_a + half / 2;
    const uint64_t deadline = global_timer_ns() + a.timeout_ns;
    const T *in = (const T *)a.in;
    T *out = (T *)a.out;
    const uint64_t first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (uint64_t)gridDim.x * blockDim.x;
    auto load_blk = [&](const T *base, uint64_t line) {
        Pay8<T> v;
        const uint64_t e0 = line * E;
        if ((((uintptr_t)base) & 7) == 0 && e0 + E <= a.count) v.u = *(const uint2 *)(base + e0);
        else {
            v.u = make_uint2(0, 0);
            for (int k = 0; k < E; ++k)
                if (e0 + k < a.count) v.e[k] = base[e0 + k];
        }
        return v;
    };
    auto store_blk = [&](T *base, uint64_t line, Pay8<T> r) {
        const uint64_t e0 = line * E;
        if ((((uintptr_t)base) & 7) == 0 && e0 + E <= a.count) *(uint2 *)(base + e0) = r.u;
        else
            for (int k = 0; k < E; ++k)
                if (e0 + k < a.count) base[e0 + k] = r.e[k];
    };
    bool failed = false;
    if (rs) {
        for (uint64_t idx = first; idx < bl * (uint64_t)p; idx += stride) {
            const int q = (int)(idx / bl);
            if (q == me) continue;
            const uint64_t line = idx - (uint64_t)q * bl;
            Pay8<T> v = load_blk(in + (uint64_t)q * a.count, line);
            st_line(a.ll[q] + base_a + (uint64_t)me * piece + line * 16, v.u.x, v.u.y, a.tag);
        }
        for (uint64_t line = first; line < bl && !failed; line += stride) {
            Pay8<T> mine = load_blk(in + (uint64_t)me * a.count, line);
            Acc acc[E];
            for (int q = 0; q < p && !failed; ++q) {
                Pay8<T> v;
                if (q == me) v = mine;
                else {
                    uint4 l;
                    if (!ll_poll(a, a.ll[me] + base_a + (uint64_t)q * piece + line * 16, deadline, q, l)) { failed = true; break; }
                    v.u = make_uint2(l.x, l.z);
                }
                if (q == 0) {
#pragma unroll
                    for (int k = 0; k < E; ++k) acc[k] = N::up(v.e[k]);
                } else {
#pragma unroll
                    for (int k = 0; k < E; ++k) acc[k] = ll_op<OP>(acc[k], N::up(v.e[k]));
                }
            }
            if (failed) break;
            Pay8<T> r;
#pragma unroll
            for (int k = 0; k < E; ++k) r.e[k] = N::down(acc[k]);
            store_blk(out, line, r);
        }
    } else {
        T *own = out + (uint64_t)me * a.count;
        for (uint64_t line = first; line < bl; line += stride) {
            Pay8<T> v = load_blk(in, line);
            for (int i = 1; i < p; ++i) {
                int q = me + i;
                if (q >= p) q -= p;
                st_line(a.ll[q] + base_b + (uint64_t)me * piece + line * 16, v.u.x, v.u.y, a.tag);
            }
            if ((const T *)own != in) store_blk(own, line, v);
        }
        for (uint64_t idx = first; idx < bl * (uint64_t)p && !failed; idx += stride) {
            const int q = (int)(idx / bl);
            if (q == me) continue;
            const uint64_t line = idx - (uint64_t)q * bl;
            uint4 l;
            if (!ll_poll(a, a.ll[me] + base_b + (uint64_t)q * piece + line * 16, deadline, q, l)) { failed = true; break; }
            Pay8<T> r;
            r.u = make_uint2(l.x, l.z);
            store_blk(out + (uint64_t)q * a.count, line, r);
        }
    }
    if (failed) return;  // head stays ahead of tail: the heartbeat reports the op as stuck / failed
    __syncthreads();
    if (threadIdx.x == 0 && a.exit_counter) {
        __threadfence();
        if (atomicAdd(a.exit_counter, 1u) == gridDim.x - 1) {
            *a.exit_counter = 0;
            *a.dev_tail = a.exe_id;
        }
    }
}

template <class T> const void *ll_kernel_of(int op, uint32_t kind)
{
    const bool two_shot = kind == LL_AR_TWOSHOT;
    if (kind == LL_REDUCE_SCATTER || kind == LL_ALLGATHER) {
        switch (kind == LL_ALLGATHER ? (int)HCCL_REDUCE_SUM : op) {  // AllGather reduces nothing: one instance serves it
            case HCCL_REDUCE_SUM: return (const void *)ll_rsag_kernel<T, HCCL_REDUCE_SUM>;
            case HCCL_REDUCE_PROD: return (const void *)ll_rsag_kernel<T, HCCL_REDUCE_PROD>;
            case HCCL_REDUCE_MAX: return (const void *)ll_rsag_kernel<T, HCCL_REDUCE_MAX>;
            default: return (const void *)ll_rsag_kernel<T, HCCL_REDUCE_MIN>;
        }
    }
    if (two_shot) {
        switch (op) {
            case HCCL_REDUCE_SUM: return (const void *)ar_ll2_kernel<T, HCCL_REDUCE_SUM>;
            case HCCL_REDUCE_PROD: return (const void *)ar_ll2_kernel<T, HCCL_REDUCE_PROD>;
            case HCCL_REDUCE_MAX: return (const void *)ar_ll2_kernel<T, HCCL_REDUCE_MAX>;
            default: return (const void *)ar_ll2_kernel<T, HCCL_REDUCE_MIN>;
        }
    }
    switch (op) {
        case HCCL_REDUCE_SUM: return (const void *)ar_ll_kernel<T, HCCL_REDUCE_SUM>;
        case HCCL_REDUCE_PROD: return (const void *)ar_ll_kernel<T, HCCL_REDUCE_PROD>;
        case HCCL_REDUCE_MAX: return (const void *)ar_ll_kernel<T, HCCL_REDUCE_MAX>;
        default: return (const void *)ar_ll_kernel<T, HCCL_REDUCE_MIN>;
    }
}

}  // namespace

HcclResult launch_ar_ll(const LlArgs *args, int nlocal, int dtype, int op, void *stream)
{
    const void *fn = nullptr;
    const uint32_t two = args[0].two_shot;  // LlKind
    switch (dtype) {
        case HCCL_DATA_TYPE_INT8: fn = ll_kernel_of<int8_t>(op, two); break;
        case HCCL_DATA_TYPE_UINT8: fn = ll_kernel_of<uint8_t>(op, two); break;
        case HCCL_DATA_TYPE_INT16: fn = ll_kernel_of<int16_t>(op, two); break;
        case HCCL_DATA_TYPE_UINT16: fn = ll_kernel_of<uint16_t>(op, two); break;
        case HCCL_DATA_TYPE_INT32: fn = ll_kernel_of<int32_t>(op, two); break;
        case HCCL_DATA_TYPE_UINT32: fn = ll_kernel_of<uint32_t>(op, two); break;
        case HCCL_DATA_TYPE_INT64: fn = ll_kernel_of<long long>(op, two); break;
        case HCCL_DATA_TYPE_UINT64: fn = ll_kernel_of<unsigned long long>(op, two); break;
        case HCCL_DATA_TYPE_FP32: fn = ll_kernel_of<float>(op, two); break;
        case HCCL_DATA_TYPE_FP64: fn = ll_kernel_of<double>(op, two); break;
        case HCCL_DATA_TYPE_FP16: fn = ll_kernel_of<__half>(op, two); break;
        case HCCL_DATA_TYPE_BFP16: fn = ll_kernel_of<__nv_bfloat16>(op, two); break;
        default: return HCCL_E_NOT_SUPPORT;
    }
    if (nlocal < 1 || nlocal > kMaxRanks) return HCCL_E_PARA;
    LlArgsArray arr;
    for (int i = 0; i < nlocal; ++i) arr.a[i] = args[i];
    int es = dtype_size(dtype);
    // lines a rank handles: the message (AllReduce), or the p blocks that pass through its hands (ReduceScatter / AllGather)
    uint64_t nlines = (args[0].count * es + 7) / 8 * (two >= LL_REDUCE_SCATTER ? (uint64_t)args[0].nranks : 1);
    unsigned ctas = (unsigned)((nlines + kLlThreads - 1) / kLlThreads);
    unsigned cap = nlocal > 1 ? (unsigned)(128 / nlocal) : (two ? 128u : 96u);
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    dim3 grid(ctas, (unsigned)nlocal), block(kLlThreads);
    void *kargs[] = {(void *)&arr};
    cudaError_t e = nlocal > 1 ? cudaLaunchCooperativeKernel(fn, grid, block, kargs, 0, (cudaStream_t)stream)
                               : cudaLaunchKernel(fn, grid, block, kargs, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        HLOG_ERROR("LL allreduce launch failed: %s", cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
