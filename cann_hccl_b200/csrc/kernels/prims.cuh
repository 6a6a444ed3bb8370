// Device primitives shared by all kernels: system-scope flag stores / loads, bounded waits, streaming loads,
// NVLS multimem accesses.  Every wait in the library goes through wait_flag_ge so that no kernel can spin without
// a bound: it ends when the flag arrives, when the deadline (globaltimer) passes, when the host raises the abort
// word, or when another CTA of the same rank has already failed.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "algo/plan.h"

namespace hcclb {

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(uint64_t *p, uint64_t v)
{
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_relaxed_sys(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// 16-byte load that does not allocate in L1: staging buffers are rewritten by peers between ops
__device__ __forceinline__ uint4 ld_stream(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void multimem_st_v4(uint8_t *mc, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// 16 bytes reduced inside the switch over all ranks' copies
template <class T, int OP> __device__ __forceinline__ uint4 multimem_ld_reduce(const uint8_t *mc);
template <> __device__ __forceinline__ uint4 multimem_ld_reduce<float, HCCL_REDUCE_SUM>(const uint8_t *mc)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
#define HCCLB_MC_HALF(T, SUF)                                                                                                             \
    template <> __device__ __forceinline__ uint4 multimem_ld_reduce<T, HCCL_REDUCE_SUM>(const uint8_t *mc)                               \
    {                                                                                                                                     \
        uint4 v;                                                                                                                          \
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4." SUF " {%0,%1,%2,%3}, [%4];"                                 \
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                                                  \
        return v;                                                                                                                         \
    }                                                                                                                                     \
    template <> __device__ __forceinline__ uint4 multimem_ld_reduce<T, HCCL_REDUCE_MAX>(const uint8_t *mc)                               \
    {                                                                                                                                     \
        uint4 v;                                                                                                                          \
        asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4." SUF " {%0,%1,%2,%3}, [%4];"                                          \
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                                                  \
        return v;                                                                                                                         \
    }                                                                                                                                     \
    template <> __device__ __forceinline__ uint4 multimem_ld_reduce<T, HCCL_REDUCE_MIN>(const uint8_t *mc)                               \
    {                                                                                                                                     \
        uint4 v;                                                                                                                          \
        asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4." SUF " {%0,%1,%2,%3}, [%4];"                                          \
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                                                  \
        return v;                                                                                                                         \
    }
HCCLB_MC_HALF(__half, "f16x2")
HCCLB_MC_HALF(__nv_bfloat16, "bf16x2")
#undef HCCLB_MC_HALF
// 32-bit integers: multimem.ld_reduce has no vector form for them, four scalar reductions per 16 bytes
#define HCCLB_MC_INT(T, OPC, OPS, SUF)                                                                             \
    template <> __device__ __forceinline__ uint4 multimem_ld_reduce<T, OPC>(const uint8_t *mc)                    \
    {                                                                                                              \
        uint4 v;                                                                                                   \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." OPS "." SUF " %0, [%1];" : "=r"(v.x) : "l"(mc) : "memory");      \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." OPS "." SUF " %0, [%1];" : "=r"(v.y) : "l"(mc + 4) : "memory");  \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." OPS "." SUF " %0, [%1];" : "=r"(v.z) : "l"(mc + 8) : "memory");  \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." OPS "." SUF " %0, [%1];" : "=r"(v.w) : "l"(mc + 12) : "memory"); \
        return v;                                                                                                  \
    }
HCCLB_MC_INT(int32_t, HCCL_REDUCE_SUM, "add", "s32")
HCCLB_MC_INT(int32_t, HCCL_REDUCE_MAX, "max", "s32")
HCCLB_MC_INT(int32_t, HCCL_REDUCE_MIN, "min", "s32")
HCCLB_MC_INT(uint32_t, HCCL_REDUCE_SUM, "add", "u32")
HCCLB_MC_INT(uint32_t, HCCL_REDUCE_MAX, "max", "u32")
HCCLB_MC_INT(uint32_t, HCCL_REDUCE_MIN, "min", "u32")
#undef HCCLB_MC_INT

struct WaitCtx {
    uint64_t deadline;             // globaltimer value after which a wait gives up
    volatile uint32_t *abort;      // host-mapped abort word (1 = suspend requested, 2 = a peer failed)
    uint32_t *local_fail;          // device word set by the first CTA of this rank that fails
};

// Spin until *flag >= want.  Returns 0, HCCL_E_TIMEOUT, HCCL_E_SUSPENDING or HCCL_E_REMOTE.
__device__ __forceinline__ int wait_flag_ge(const uint64_t *flag, uint64_t want, const WaitCtx &w, uint64_t &seen)
{
    for (uint32_t it = 0;; ++it) {
        seen = ld_acquire_sys(flag);
        if (seen >= want) return 0;
        if ((it & 127) == 127) {
            if (global_timer_ns() > w.deadline) return HCCL_E_TIMEOUT;
            if (w.local_fail && *(volatile uint32_t *)w.local_fail) return (int)*(volatile uint32_t *)w.local_fail;
            if ((it & 4095) == 4095 && w.abort) {
                uint32_t ab = *w.abort;
                if (ab) return ab == 2 ? HCCL_E_REMOTE : HCCL_E_SUSPENDING;
            }
        }
    }
}

// First failure of a rank wins: fills the host-mapped status block.
__device__ __forceinline__ void report_failure(const RankCtx &c, uint64_t seq, int code, int step, int peer, int chan, uint64_t want,
                                               uint64_t seen)
{
    if (atomicCAS(c.exit_counter + 1, 0u, (uint32_t)code) != 0u) return;
    DevStatus *s = c.status;
    s->step = (uint32_t)step;
    s->peer = peer;
    s->chan = (uint32_t)chan;
    s->expected = want;
    s->seen = seen;
    s->seq = seq;
    __threadfence_system();
    *(volatile uint32_t *)&s->code = (uint32_t)code;
}

}  // namespace hcclb
