// Overflow scan: counts the Inf / NaN elements of a floating-point buffer into a host-mapped counter.  Launched after a
// reduction when HCCL_OVERFLOW_CHECK=1 (role of the reference's overflow-detection address hookup,
// common/debug/profiling/task_overflow.cc: there the hardware flags saturation, here the output is inspected).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include "common/base.h"
#include "hccl/hccl_types.h"
#include "kernels/overflow.h"

namespace hcclb {

template <typename T> __device__ __forceinline__ bool bad_value(T v);
template <> __device__ __forceinline__ bool bad_value<float>(float v) { return !isfinite(v); }
template <> __device__ __forceinline__ bool bad_value<double>(double v) { return !isfinite(v); }
template <> __device__ __forceinline__ bool bad_value<__half>(__half v) { return !isfinite(__half2float(v)); }
template <> __device__ __forceinline__ bool bad_value<__nv_bfloat16>(__nv_bfloat16 v) { return !isfinite(__bfloat162float(v)); }

template <typename T> __global__ void overflow_scan_kernel(const T *buf, uint64_t n, unsigned long long *counter)
{
    unsigned long long mine = 0;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) mine += bad_value(buf[i]) ? 1 : 0;
    // warp, then block, then one system-scope atomic per block that saw something
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_down_sync(0xffffffffu, mine, o);
    __shared__ unsigned long long part[32];
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long total = 0;
        for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w) total += part[w];
        if (total) atomicAdd_system(counter, total);
    }
}

HcclResult launch_overflow_scan(const void *buf, uint64_t count, int dtype, unsigned long long *counter, void *stream)
{
    if (count == 0) return HCCL_SUCCESS;
    cudaStream_t st = (cudaStream_t)stream;
    int blocks = (int)std::min<uint64_t>(296, (count + 255) / 256);
    switch (dtype) {
        case HCCL_DATA_TYPE_FP32: overflow_scan_kernel<float><<<blocks, 256, 0, st>>>((const float *)buf, count, counter); break;
        case HCCL_DATA_TYPE_FP64: overflow_scan_kernel<double><<<blocks, 256, 0, st>>>((const double *)buf, count, counter); break;
        case HCCL_DATA_TYPE_FP16: overflow_scan_kernel<__half><<<blocks, 256, 0, st>>>((const __half *)buf, count, counter); break;
        case HCCL_DATA_TYPE_BFP16: overflow_scan_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16 *)buf, count, counter); break;
        default: return HCCL_SUCCESS;  // integers cannot hold Inf / NaN
    }
    return cudaGetLastError() == cudaSuccess ? HCCL_SUCCESS : HCCL_E_RUNTIME;
}

}  // namespace hcclb
