// Schedule generators: lower (collective, algorithm, sizes) to a Plan.
// Patterns follow the algorithm families of the reference's template layer
// (algorithm/base/alg_template/**: ring, mesh, halving-doubling with non-power-of-two fold,
// pairwise, star) but are expressed in pull form over peer-mapped staging, with flag waits in place
// of the TxAck/RxAck/TxAsync/RxAsync link verbs.
#pragma once
#include <string>
#include <vector>
#include "algo/plan.h"

namespace hcclb {

enum CollType : int {
    COLL_ALLREDUCE = 0, COLL_BROADCAST, COLL_REDUCE_SCATTER, COLL_REDUCE_SCATTER_V, COLL_SCATTER,
    COLL_ALLGATHER, COLL_ALLGATHER_V, COLL_BARRIER, COLL_ALLTOALL, COLL_ALLTOALLV, COLL_ALLTOALLVC,
    COLL_REDUCE, COLL_GATHER, COLL_SEND, COLL_RECV, COLL_BATCH_SENDRECV, COLL_COUNT
};
const char *coll_name(int coll);

enum AlgoId : int {
    ALGO_AUTO = 0,
    ALGO_MESH,          // AllReduce: two-shot (reduce-scatter + all-gather over all peers); others: one round over all peers
    ALGO_MESH_ONESHOT,  // AllReduce only: every rank reduces the whole message
    ALGO_RING,
    ALGO_RHD,           // recursive halving-doubling, non-power-of-two ranks folded
    ALGO_PAIRWISE,      // AlltoAll family
    ALGO_STAR,          // rooted ops: root talks to every peer directly
    ALGO_TREE,          // rooted ops: binomial tree
    ALGO_NVLS,          // in-switch reduction / multicast (two-shot for AllReduce)
    ALGO_NVLS_ONESHOT,  // AllReduce: multimem.ld_reduce of the whole message on every rank
    ALGO_SINGLE,        // one rank: local copy
    ALGO_MESH_PIPE,     // AllReduce / ReduceScatter / AllGather / Broadcast: pipelined kernel (kernels/pipe_coll.*), CTA stages over a ring of
                        // staging slots, peer loads and stores; no step list (device only; CPU ranks run the plain mesh / ring schedule)
    ALGO_NVLS_PIPE,     // same with in-switch reduction (multimem.ld_reduce) and multicast stores
    ALGO_NVLS_ZC,       // AllReduce on registered symmetric buffers: multimem.ld_reduce from the send buffers, multimem.st into the receive buffers, no staging
    ALGO_LL,            // AllReduce, small messages: data and flag travel together in 16-byte lines (device only)
    ALGO_MESH_ZC,       // AllReduce (two ranks) / ReduceScatter / AllGather on a registered send buffer: peers read it in place (kernels/pipe_coll.*)
    ALGO_DIRECT,        // AlltoAll family: parametric kernel, counts travel as launch arguments (kernels/a2av.cu; device only)
    ALGO_COUNT
};
const char *algo_name(int algo);
int algo_from_name(const std::string &name);  // ALGO_AUTO when unknown

struct OpDesc {
    int coll = COLL_ALLREDUCE;
    int algo = ALGO_MESH;
    int nranks = 1;
    int root = 0;
    int dtype = HCCL_DATA_TYPE_FP32;
    int redop = HCCL_REDUCE_SUM;
    int nchan = 1;
    uint64_t count = 0;        // per-API element count (AllReduce count, AllGather sendCount, ReduceScatter recvCount, ...)
    uint64_t chunk_off = 0;    // window of `count` this plan covers (staging loop)
    uint64_t chunk_count = 0;
    uint64_t slot_bytes = 0;   // AlltoAllV: bytes of one per-sender staging slot
    // V variants (arrays of nranks entries, elements).  AllGatherV: counts/displs describe the receive
    // layout; ReduceScatterV: the send layout.  AlltoAllV: this rank's four rows, only valid for
    // plans built for a single local rank; AlltoAllVC and emulated ranks pass the full matrix instead.
    std::vector<uint64_t> counts, displs;
    std::vector<uint64_t> send_counts, send_displs, recv_counts, recv_displs;  // [local][nranks] flattened
    int peer = -1;             // Send/Recv: remote rank
    uint32_t p2p_round0 = 0;   // Send/Recv: rounds already exchanged on this ordered pair
    uint64_t p2p_slot = 0;     // Send/Recv: mailbox slot bytes
};

// Build the plan for the ranks listed in `local` (their step lists are stored in that order).
// Returns HCCL_E_NOT_SUPPORT when the algorithm does not exist for the collective.
HcclResult build_plan(const OpDesc &d, const std::vector<int> &local, Plan *plan);

// Staging bytes per rank that `chunk_count` elements need under this algorithm (to size the staging loop).
uint64_t plan_stage_bytes(const OpDesc &d);

// Static bounds check of a plan built from `d` for the ranks `local`: operand ranges against the declared staging need
// (and one staging half when stage_half != 0), the mailbox area and the caller's buffer sizes that the API contract implies;
// channel, bank and rank fields against their ranges.  HCCL_E_INTERNAL and a description in *why on the first violation.
HcclResult verify_plan(const OpDesc &d, const std::vector<int> &local, const Plan &plan, uint64_t stage_half, std::string *why);

// Static race detection of a plan built for ALL ranks of `d` (algo/racecheck.cc): any two accesses to overlapping bytes of one
// buffer, one of them a write, must be ordered by program order and flag waits; unsatisfiable waits and cycles are reported too.
// `in_place` folds each rank's send and receive buffer into one, as the in-place form of the collective lays them out.
HcclResult race_check_plan(const OpDesc &d, const Plan &plan, bool in_place, std::string *why);

}  // namespace hcclb
