// Launcher of the pipelined large-message kernels (pipe_coll.cuh); the kernels themselves are instantiated per element
// type in exec_plan_<type>.cu.
#include <cuda_runtime.h>
#include <mutex>
#include <set>
#include <utility>
#include "common/log.h"
#include "kernels/pipe_coll.h"

namespace hcclb {

constexpr int kPipeThreads = 512;

const void *pipe_kernel_i8(int op);
const void *pipe_kernel_u8(int op);
const void *pipe_kernel_i16(int op);
const void *pipe_kernel_u16(int op);
const void *pipe_kernel_i32(int op);
const void *pipe_kernel_u32(int op);
const void *pipe_kernel_i64(int op);
const void *pipe_kernel_u64(int op);
const void *pipe_kernel_f32(int op);
const void *pipe_kernel_f64(int op);
const void *pipe_kernel_f16(int op);
const void *pipe_kernel_bf16(int op);

static const void *pipe_kernel_for(int dtype, int op)
{
    switch (dtype) {
        case HCCL_DATA_TYPE_INT8: return pipe_kernel_i8(op);
        case HCCL_DATA_TYPE_UINT8: return pipe_kernel_u8(op);
        case HCCL_DATA_TYPE_INT16: return pipe_kernel_i16(op);
        case HCCL_DATA_TYPE_UINT16: return pipe_kernel_u16(op);
        case HCCL_DATA_TYPE_INT32: return pipe_kernel_i32(op);
        case HCCL_DATA_TYPE_UINT32: return pipe_kernel_u32(op);
        case HCCL_DATA_TYPE_INT64: return pipe_kernel_i64(op);
        case HCCL_DATA_TYPE_UINT64: return pipe_kernel_u64(op);
        case HCCL_DATA_TYPE_FP32: return pipe_kernel_f32(op);
        case HCCL_DATA_TYPE_FP64: return pipe_kernel_f64(op);
        case HCCL_DATA_TYPE_FP16: return pipe_kernel_f16(op);
        case HCCL_DATA_TYPE_BFP16: return pipe_kernel_bf16(op);
        default: return pipe_kernel_u8(HCCL_REDUCE_SUM);  // transport-only types: AllGather / Broadcast only copy
    }
}

HcclResult launch_pipe_coll(const RankCtx *dev_ctx, const PipeArgs *args, int nlocal, int redop, void *stream)
{
    if (nlocal < 1 || nlocal > kMaxRanks) return HCCL_E_PARA;
    const PipeArgs &a0 = args[0];
    if (a0.mode < 0 || a0.mode >= PM_COUNT) return HCCL_E_PARA;
    const bool bcast = pipe_mode_is_bcast(a0.mode), three = pipe_mode_has_copy_out(a0.mode);
    const int nb = bcast ? a0.n1 : a0.n1 + a0.n2 + (three ? a0.n3 : 0);
    if (nb < 1 || nb > kMaxChannels || a0.nslots < 1 || a0.nslots > kPipeMaxSlots || a0.chunk_elems == 0) return HCCL_E_PARA;
    if (a0.n1 < 1 || (!bcast && a0.n2 < 1) || (three && a0.n3 < 1)) return HCCL_E_PARA;
    if (pipe_mode_is_zc(a0.mode) && !a0.z_in_peer) return HCCL_E_PARA;
    if (a0.g1 < 1 || a0.g2 < 1 || a0.g3 < 1) return HCCL_E_PARA;
    PipeArgsArray arr;
    for (int i = 0; i < nlocal; ++i) arr.a[i] = args[i];
    const void *fn = pipe_kernel_for(a0.dtype, redop);
    {
        // the opt-in to more than 48 KB of dynamic shared memory is a property of (device, function): once for each pair
        static std::mutex mu;
        static std::set<std::pair<int, const void *>> done;
        int dev = 0;
        cudaGetDevice(&dev);
        std::lock_guard<std::mutex> lk(mu);
        if (!done.count({dev, fn})) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPipeDynSmem);
            if (e != cudaSuccess) {
                HLOG_ERROR("cudaFuncSetAttribute(pipelined kernel, %zu bytes of shared memory) failed: %s", kPipeDynSmem, cudaGetErrorString(e));
                return HCCL_E_RUNTIME;
            }
            done.insert({dev, fn});
        }
    }
    dim3 grid((unsigned)nb, (unsigned)nlocal), block(kPipeThreads);
    void *kargs[] = {(void *)&dev_ctx, (void *)&arr};
    cudaError_t e = cudaLaunchCooperativeKernel(fn, grid, block, kargs, kPipeDynSmem, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        HLOG_ERROR("pipelined kernel launch failed (mode %d, grid %dx%d): %s", a0.mode, nb, nlocal, cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
