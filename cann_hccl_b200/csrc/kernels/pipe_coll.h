// Launch interface of the pipelined large-message kernels (kernels/pipe_coll.cuh, pipe_coll.cu).
//
// One launch runs a whole collective of any size through a small ring of staging slots: the message is cut into
// chunks, and the CTAs of a rank are split into groups that each own one stage of the pipeline (copy-in, transfer /
// reduce over NVLink, copy-out), so that the local copies of chunk c+1 and c-1 run while chunk c crosses the links.
// Role of the reference's big-data AIV kernels (algorithm/base/alg_aiv_template/aiv_all_reduce_910b_bigdata.h:19-127
// ReduceWithFlagWrap, aiv_all_gather_910b_bigdata.h:74-154 MemcpyWithFlagWrap, aiv_reduce_scatter_910b_bigdata.h),
// which overlap producer and consumer blocks with progress flags.
#pragma once
#include "algo/plan.h"

namespace hcclb {

enum PipeMode : int32_t {
    PM_ALLREDUCE = 0,      // two-shot: copy-in | reduce my slice of the chunk over all ranks, write it back to all | copy-out
    PM_ALLREDUCE_ONESHOT,  // copy-in | every rank reduces the whole chunk from all slots straight into its receive buffer
    PM_REDUCE_SCATTER,     // copy-in of the p blocks of a chunk | reduce my block over all ranks into the receive buffer
    PM_ALLGATHER,          // copy-in of my block | pull the peers' blocks straight into the receive buffer
    PM_BROADCAST_MC,       // root: multicast store of the chunk into every rank's slot | others: copy-out
    PM_BROADCAST_CHAIN,    // root -> root+1 -> ... : every rank pulls the chunk from its predecessor's slot
};

constexpr int kPipeMaxSlots = 16;
constexpr int kPipeRoles = 3;
constexpr size_t kPipeCounterWords = (size_t)kPipeRoles * kPipeMaxSlots;  // per local rank, device memory, zero between ops
// Flag words of the pipeline inside bank 0 of the flag page (channel index): values are (seq << kSeqShift) + chunk + 1.
constexpr int kPipeWordReady = 0;  // source rank finished staging the chunk
constexpr int kPipeWordDone = 1;   // source rank finished its transfer stage on the chunk
constexpr int kPipeWordOut = 2;    // (own page only) copy-out of the chunk finished
constexpr int kPipeTraceWords = 16;

struct PipeArgs {
    const uint8_t *in;
    uint8_t *out;
    uint64_t count;        // elements: AllReduce / Broadcast message, AllGather send count, ReduceScatter receive count
    uint64_t chunk_elems;  // elements of one block that a chunk covers
    uint64_t seq;
    int32_t mode, dtype, root, nslots;
    int32_t n1, n2, n3;    // CTAs per stage (AllReduce uses all three, the other modes the first two; Broadcast: all CTAs do one job)
    int32_t use_mc;        // 1: multimem.ld_reduce / multimem.st through the NVLS mapping of the staging buffer
};
struct PipeArgsArray {
    PipeArgs a[kMaxRanks];
};

// Bytes of one ring slot for the given mode.
HCCLB_HD uint64_t pipe_slot_bytes(int mode, uint64_t chunk_elems, int es, int p)
{
    return (mode == PM_REDUCE_SCATTER ? (uint64_t)p : 1ull) * chunk_elems * (uint64_t)es;
}

// One launch runs the listed local ranks (more than one: virtual ranks of one GPU).  Always a cooperative launch: the
// stages of a rank wait on one another, so all CTAs have to be resident together.
HcclResult launch_pipe_coll(const RankCtx *dev_ctx, const PipeArgs *args, int nlocal, int redop, void *stream);

}  // namespace hcclb
