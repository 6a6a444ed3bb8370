// Launch interface of the parametric AlltoAll / AlltoAllV / AlltoAllVC kernel (kernels/a2av.cu).
//
// Counts and displacements travel as kernel arguments, so a call with a new count matrix builds nothing, allocates
// nothing and copies nothing to the device beforehand (the step-list plans of the same collectives bake the counts into
// their steps).  The reference plans AlltoAllV from a count matrix exchanged on the host for every call
// (framework/communicator/impl/hccl_communicator.cc:3928, algorithm/base/alg_template/temp_alltoallv/alltoallv_pairwise.cc:72-283);
// here each ordered pair of ranks runs its own flow-controlled stream and needs no global view.
#pragma once
#include "algo/plan.h"

namespace hcclb {

constexpr int kA2avMaxLanes = 32;

struct A2avArgs {
    const uint8_t *in;
    uint8_t *out;
    uint64_t send_counts[kMaxRanks], send_displs[kMaxRanks];  // elements, by destination rank
    uint64_t recv_counts[kMaxRanks], recv_displs[kMaxRanks];  // elements, by source rank
    uint64_t seq;
    uint64_t sub_bytes;   // bytes of one of the two sub-slots that a (source rank, lane) pair owns in the receiver's staging half
    int32_t dtype, lanes;
};
struct A2avArgsArray {
    A2avArgs a[kMaxRanks];
};

// Staging bytes a rank needs: every source rank x lane owns two sub-slots.
HCCLB_HD uint64_t a2av_stage_bytes(int p, int lanes, uint64_t sub_bytes) { return (uint64_t)p * lanes * 2 * sub_bytes; }

// One launch runs the listed local ranks (more than one: virtual ranks of one GPU, cooperative launch).
HcclResult launch_a2av(const RankCtx *dev_ctx, const A2avArgs *args, int nlocal, int nranks, void *stream);

}  // namespace hcclb
