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

namespace hcclb {

constexpr int kExecThreads = 512;
struct ExecArgsArray {
    ExecArgs a[kMaxRanks];
};

const void *exec_kernel_i8(int op);
const void *exec_kernel_u8(int op);
const void *exec_kernel_i16(int op);
const void *exec_kernel_u16(int op);
const void *exec_kernel_i32(int op);
const void *exec_kernel_u32(int op);
const void *exec_kernel_i64(int op);
const void *exec_kernel_u64(int op);
const void *exec_kernel_f32(int op);
const void *exec_kernel_f64(int op);
const void *exec_kernel_f16(int op);
const void *exec_kernel_bf16(int op);

static const void *exec_kernel_for(int dtype, int op)
{
    switch (dtype) {
        case HCCL_DATA_TYPE_INT8: return exec_kernel_i8(op);
        case HCCL_DATA_TYPE_UINT8: return exec_kernel_u8(op);
        case HCCL_DATA_TYPE_INT16: return exec_kernel_i16(op);
        case HCCL_DATA_TYPE_UINT16: return exec_kernel_u16(op);
        case HCCL_DATA_TYPE_INT32: return exec_kernel_i32(op);
        case HCCL_DATA_TYPE_UINT32: return exec_kernel_u32(op);
        case HCCL_DATA_TYPE_INT64: return exec_kernel_i64(op);
        case HCCL_DATA_TYPE_UINT64: return exec_kernel_u64(op);
        case HCCL_DATA_TYPE_FP32: return exec_kernel_f32(op);
        case HCCL_DATA_TYPE_FP64: return exec_kernel_f64(op);
        case HCCL_DATA_TYPE_FP16: return exec_kernel_f16(op);
        case HCCL_DATA_TYPE_BFP16: return exec_kernel_bf16(op);
        default: return exec_kernel_u8(HCCL_REDUCE_SUM);  // transport-only types: plans contain copies only
    }
}

HcclResult launch_exec_plan(const RankCtx *dev_ctx, const ExecArgs *args, int nlocal, int nchan, void *stream, bool co_resident)
{
    if (nlocal < 1 || nlocal > kMaxRanks || nchan < 1 || nchan > kMaxChannels) return HCCL_E_PARA;
    ExecArgsArray arr;
    for (int i = 0; i < nlocal; ++i) arr.a[i] = args[i];
    dim3 grid((unsigned)nchan, (unsigned)nlocal), block(kExecThreads);
    const void *fn = exec_kernel_for(args[0].dtype, args[0].redop);
    void *kargs[] = {(void *)&dev_ctx, (void *)&arr};
    cudaError_t e;
    // Virtual ranks of one GPU wait on one another, and some plans make a rank's CTAs wait on each other (a barrier over
    // its own channels, CTA groups handing chunks on): all those CTAs must be resident at the same time, or a waiting CTA
    // could occupy the SM that the CTA it waits for needs while another kernel holds the rest of the GPU.  A cooperative
    // launch guarantees the co-residency (and fails at launch when the grid cannot fit).
    if (nlocal > 1 || co_resident) e = cudaLaunchCooperativeKernel(fn, grid, block, kargs, 0, (cudaStream_t)stream);
    else e = cudaLaunchKernel(fn, grid, block, kargs, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        HLOG_ERROR("executor launch failed (grid %dx%d): %s", nchan, nlocal, cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
