// Plan IR: every collective algorithm is lowered by the schedule generators to a short per-rank list
// of steps.  The same list is interpreted by the sm_100a executor kernel (one CTA per channel, peers'
// staging reached through NVLink peer mappings or the NVLS multicast mapping) and by the host-memory
// transport (CPU ranks, shared memory).  This replaces the reference's executor -> template ->
// dispatcher-task layering (algorithm/impl/coll_executor/**, algorithm/base/alg_template/**): a step is
// the analogue of one {notify wait, SDMA copy / inline reduce, notify record} task group.
#pragma once
#include <string>
#include <vector>
#include "common/base.h"

namespace hcclb {

enum StepOp : uint8_t {
    ST_NOP = 0,         // only wait / signal
    ST_COPY = 1,        // d (and d2) = a
    ST_REDUCE2 = 2,     // d (and d2) = a (+) b
    ST_REDUCE_ALL = 3,  // d (and d2) = (+)_{q=0..p-1} a@rank q   (fixed rank order: deterministic)
    ST_GATHER_ALL = 4,  // for q: d[q*d_stride ..] = a@rank q [q*a_stride ..]; block q holds
                        //        clamp(limit - q*count, 0, count) elements when limit != 0
    ST_MC_REDUCE = 5,   // d (and d2) = multimem.ld_reduce over the NVLS mapping of a (device only)
};

enum BufKind : uint8_t {
    BUF_IN = 0,     // caller's send buffer (only addressable on its own rank)
    BUF_OUT = 1,    // caller's receive buffer
    BUF_STAGE = 2,  // this op's half of the peer-mapped staging buffer
    BUF_P2P = 3,    // peer-mapped mailbox area used by Send/Recv on the host / emulated transports
    BUF_ZIN = 4,    // caller's send buffer inside registered symmetric memory: addressable on every rank (zero-copy)
    BUF_ZOUT = 5,   // caller's receive buffer inside registered symmetric memory
    BUF_NONE = 7,
};

constexpr int16_t RANK_SELF = -1;  // buffer of the executing rank
constexpr int16_t RANK_NONE = -1;  // no wait / no signal
constexpr int16_t RANK_ALL = -2;   // every other rank (wait / signal), or the NVLS multicast mapping (d_rank)

enum StepFlags : uint8_t {
    SF_SKIP_SELF = 1,   // GATHER_ALL: do not copy the executing rank's own block
    SF_WAIT_ALLCH = 2,  // wait for every channel [wait_clo, wait_clo+wait_cn) of the producer, not only my lane
    SF_INCLUDE_SELF = 8,  // RANK_ALL waits / signals also cover the executing rank (dependencies between its own CTA groups)
    SF_ABS_VALS = 4,    // wait_val / sig_val are absolute flag values (Send/Recv), not relative to the op sequence
};

struct Step {
    uint8_t op;
    uint8_t flags;
    uint8_t a_buf, b_buf, d_buf, d2_buf;
    uint8_t wait_bank, sig_bank;
    int16_t a_rank, b_rank, d_rank;  // owner of the buffer; d2 is always local
    int16_t wait_rank, sig_rank;     // RANK_NONE / RANK_ALL / rank
    uint16_t chan_lo, chan_n;        // channels executing this step; data is split evenly among them
    uint16_t wait_clo, wait_cn;      // producer channel range when SF_WAIT_ALLCH
    uint32_t wait_val, sig_val;
    uint64_t a_off, b_off, d_off, d2_off;  // bytes
    uint64_t a_stride, d_stride;           // bytes between per-rank blocks (GATHER_ALL)
    uint64_t count;                        // elements
    uint64_t limit;                        // GATHER_ALL clamp (elements), 0 = none
};

// Per-rank view of a communicator as the executors see it (device copy for kernels, host copy for CPU ranks).
struct RankCtx {
    int32_t rank, nranks;
    uint8_t *stage[kMaxRanks];   // staging buffer of rank q mapped into this rank's address space
    uint64_t *flags[kMaxRanks];  // flag page of rank q (layout: flag_index())
    uint8_t *p2p[kMaxRanks];     // p2p mailbox area of rank q
    uint8_t *ll[kMaxRanks];      // low-latency AllReduce mailboxes of rank q
    uint8_t *mc_stage;           // NVLS multicast mapping of the staging buffer (null when unavailable)
    DevStatus *status;           // host-mapped status block of this rank
    volatile uint32_t *abort;    // host-mapped abort word, non-zero = give up
    uint32_t *exit_counter;      // local counter used to find the last CTA of an op; [1] = first failure code of this rank
    uint64_t *dev_tail;          // device word: sequence number of the newest completed op
    uint64_t *trace;             // optional in-kernel timestamps (HCCL_KERNEL_TRACE=1): [0] kernel start, then 3 per step
    uint32_t *pipe_cnt;          // arrival counters of the pipelined kernels: [stage][ring slot], zero between ops
    uint64_t stage_half;         // bytes per staging half
    uint64_t timeout_ns;         // bound of every wait
};

// Arguments of one plan execution on one rank.
struct ExecArgs {
    const Step *steps;
    int32_t nsteps;
    int32_t nchan;
    uint64_t seq;          // op sequence number (ops of a communicator are numbered identically on all ranks)
    const uint8_t *in;     // BUF_IN base
    uint8_t *out;          // BUF_OUT base
    int32_t dtype, redop;
    uint32_t track_done;   // 1: collective (ping-pong halves + done flags), 0: p2p plan
    uint32_t pad;
    // zero-copy: the caller's buffers as mapped for every rank (arrays of nranks pointers) and their multicast mappings
    uint8_t *const *z_in_peer;
    uint8_t *const *z_out_peer;
    uint8_t *z_in_mc;
    uint8_t *z_out_mc;
    uint64_t z_in_off, z_out_off;  // offsets of the caller's buffers inside their symmetric allocations (peer tables hold allocation bases)
};

// Flag page layout: [bank][source rank][channel] 64-bit words, then one "done" word per source rank.
HCCLB_HD size_t flag_index(int bank, int src, int chan) { return ((size_t)bank * kMaxRanks + src) * kMaxChannels + chan; }
HCCLB_HD size_t done_index(int src) { return (size_t)kFlagBanks * kMaxRanks * kMaxChannels + src; }
constexpr int kTraceSteps = 340;  // steps whose timestamps fit the trace buffer
constexpr size_t kTraceWords = 1 + 3 * kTraceSteps;
constexpr size_t kFlagWords = (size_t)kFlagBanks * kMaxRanks * kMaxChannels + kMaxRanks;
constexpr size_t kFlagPageBytes = ((kFlagWords * 8 + 4095) / 4096) * 4096;

// Element range [lo, hi) of a step that channel `c` (relative index in the step's channel set) handles.
// Pieces are multiples of 16 bytes so that vector accesses stay aligned when the bases are.
HCCLB_HD void chan_range(uint64_t count, int esize, int cn, int c, uint64_t &lo, uint64_t &hi)
{
    uint64_t vec = esize >= 16 ? 1 : (uint64_t)(16 / esize);
    uint64_t per = round_up_u64(ceil_div_u64(count, (uint64_t)cn), vec);
    lo = per * (uint64_t)c;
    hi = lo + per;
    if (lo > count) lo = count;
    if (hi > count) hi = count;
}

// A lowered collective: the step list of each locally executed rank plus its resource needs.
struct Plan {
    std::vector<std::vector<Step>> steps;  // [local rank index]
    int nchan = 1;
    uint64_t stage_bytes = 0;  // staging bytes touched per rank (must fit one half)
    bool intra_rank_waits = false;  // some CTA of a rank waits for another CTA of the same rank: all CTAs must be resident together
    std::string name;          // "<collective>/<algorithm>"
};

}  // namespace hcclb
