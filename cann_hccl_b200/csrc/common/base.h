// Shared basic definitions for host and device code.
#pragma once
#include <stdint.h>
#include <stddef.h>
#include "hccl/hccl_types.h"

#if defined(__CUDACC__)
#define HCCLB_HD __host__ __device__ __forceinline__
#else
#define HCCLB_HD inline
#endif

namespace hcclb {

constexpr int kMaxRanks = 16;     // one NVSwitch domain (reference AIV path: MAX_RANK_SIZE 16, hccl_aiv.h:40)
constexpr int kMaxChannels = 128; // CTAs ("channels") a plan may use per rank
constexpr int kFlagBanks = 4;     // 0 data, 1 ack, 2 p2p data, 3 p2p ack
constexpr int kSeqShift = 20;     // flag value = (sequence << kSeqShift) + step value

// Byte size of one element; 0 for an unknown type.
HCCLB_HD int dtype_size(int dt)
{
    switch (dt) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_HIF8:
        case HCCL_DATA_TYPE_FP8E4M3: case HCCL_DATA_TYPE_FP8E5M2: return 1;
        case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_FP16:
        case HCCL_DATA_TYPE_BFP16: return 2;
        case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_UINT32: case HCCL_DATA_TYPE_FP32: return 4;
        case HCCL_DATA_TYPE_INT64: case HCCL_DATA_TYPE_UINT64: case HCCL_DATA_TYPE_FP64: return 8;
        case HCCL_DATA_TYPE_INT128: return 16;
        default: return 0;
    }
}

HCCLB_HD uint64_t round_up_u64(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }
HCCLB_HD uint64_t ceil_div_u64(uint64_t v, uint64_t a) { return (v + a - 1) / a; }

// Status block a device kernel (or host executor) fills when a bounded wait
// runs out or the abort word is raised.  Lives in host-mapped memory so the
// host can read it without touching the stream.
struct DevStatus {
    uint32_t code;      // HcclResult, 0 = fine
    uint32_t step;      // index of the step that gave up
    int32_t peer;       // rank whose flag was awaited
    uint32_t chan;      // channel (CTA) index
    uint64_t expected;  // flag value waited for
    uint64_t seen;      // flag value last observed
    uint64_t seq;       // op sequence number
    uint64_t head;      // op-execution counter: bumped when an op starts (first CTA)
    uint64_t tail;      // ... and when it completes (last CTA); head != tail for long = stuck
};

}  // namespace hcclb
