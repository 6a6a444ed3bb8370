// Launch interface of the pipelined large-message kernels (kernels/pipe_coll.cuh, pipe_coll.cu).
//
// One launch runs a whole collective of any size through a small ring of staging slots: the message is cut into
// chunks, and the CTAs of a rank are split into groups that each own one stage of the pipeline (stage-in or push,
// reduce / pull, copy-out), so that the local copies of chunk c+1 and c-1 run while chunk c crosses the links.
// Role of the reference's big-data AIV kernels (algorithm/base/alg_aiv_template/aiv_all_reduce_910b_bigdata.h:19-127
// ReduceWithFlagWrap, aiv_all_gather_910b_bigdata.h:74-154 MemcpyWithFlagWrap, aiv_reduce_scatter_910b_bigdata.h),
// which overlap producer and consumer blocks with progress flags.
//
// Two families.  "mc": every rank copies its chunk into its own slot, the in-switch reduction (multimem.ld_reduce)
// reads all slots at once and multimem.st writes all of them at once.  "push": a rank stores its contribution straight
// into the slots of the ranks that need it (peer stores only, no peer loads: a store needs no round trip), and every
// reduction reads local memory.
#pragma once
#include "algo/plan.h"

namespace hcclb {

enum PipeMode : int32_t {
    PM_AR2_MC = 0,  // AllReduce two-shot: copy-in | ld_reduce my slice of the chunk, multimem.st it back into every slot | copy-out
    PM_AR2_PUSH,    // AllReduce two-shot: push slice q to rank q | reduce my slice locally, store the result to every rank | copy-out
    PM_AR1_MC,      // AllReduce one-shot: copy-in | ld_reduce the whole chunk into the receive buffer
    PM_AR1_PUSH,    // AllReduce one-shot: push the chunk to every peer | reduce the p copies locally into the receive buffer
    PM_RS_MC,       // ReduceScatter: copy-in of the p blocks of a chunk | ld_reduce my block into the receive buffer
    PM_RS_PUSH,     // ReduceScatter: push block q to rank q | reduce the p copies of my block locally into the receive buffer
    PM_AG_PULL,     // AllGather: copy-in of my block | pull the peers' blocks straight into the receive buffer
    PM_BC_MC,       // Broadcast: root multicasts the chunk into every slot | the others copy out
    PM_BC_PUSH,     // Broadcast chain root -> root+1 -> ...: every rank copies its slot out and on into its successor's slot
    // zero-copy: the send buffer of every rank lies in registered symmetric memory, so the peers read it where it is.  No
    // staging and no chunks: one gate CTA tells the peers that this rank has entered the op and holds the kernel until
    // they have finished reading, the other CTAs split the whole message.
    PM_AR1_ZC,      // AllReduce one-shot: every rank reduces all p send buffers into its receive buffer (two ranks: optimal)
    PM_RS_ZC,       // ReduceScatter: every rank reduces its block of all p send buffers into its receive buffer
    PM_AG_ZC,       // AllGather: every rank pulls the peers' send buffers straight into its receive buffer
    // Reduce: the two-shot AllReduce with the reduced slices stored to the root only, which alone copies out
    PM_RD_PUSH,     // Reduce: push slice k to its owner (every rank but the root) | owners reduce, store the result to the root | root: copy-out
    PM_COUNT
};

constexpr uint32_t kTmaBuf = 32 * 1024;  // piece of a bulk asynchronous copy
constexpr int kTmaDepth = 6;             // pieces of a CTA's shared-memory ring
constexpr size_t kPipeDynSmem = (size_t)kTmaBuf * kTmaDepth;  // dynamic shared memory of the kernels
constexpr int kPipeMaxSlots = 16;
constexpr int kPipeRoles = 3;
constexpr size_t kPipeCounterWords = (size_t)kPipeRoles * kPipeMaxSlots;  // per local rank, device memory, zero between ops
// Progress words of the pipeline: one per (stage, source rank, ring slot) inside bank 0 of the flag page; the value is
// (seq << kSeqShift) + chunk + 1 of the newest chunk of that slot the stage has finished (per slot the chunks come in order).
constexpr int kPipeWordReady = 0;  // source rank finished its first stage on the chunk (slot staged, or contribution pushed)
constexpr int kPipeWordDone = 1;   // source rank finished its second stage on the chunk
constexpr int kPipeWordOut = 2;    // source rank finished copying the chunk out
HCCLB_HD size_t pipe_flag_index(int word, int src, int slot) { return flag_index(0, src, word * kPipeMaxSlots + slot); }
static_assert(kPipeRoles * kPipeMaxSlots <= kMaxChannels, "progress words must fit one bank of the flag page");

struct PipeArgs {
    const uint8_t *in;
    uint8_t *out;
    uint64_t count;        // elements: AllReduce / Broadcast message, AllGather send count, ReduceScatter receive count
    uint64_t chunk_elems;  // elements of one block that a chunk covers; a multiple of nranks * 256 bytes
    uint64_t seq;
    int32_t mode, dtype, root, nslots;
    int32_t n1, n2, n3;    // CTAs per stage (two-shot AllReduce uses all three, Broadcast only n1, the other modes the first two)
    int32_t g1, g2, g3;    // groups per stage: group g of G takes the chunks c with c % G == g (CTAs of a stage divisible by G)
    int32_t pad;
    const uint8_t *const *z_in_peer;  // zero-copy modes: device table of every rank's mapping of the registered allocation that holds `in`
    uint64_t z_in_off;                // ... and the offset of `in` inside it (the same on every rank)
};
struct PipeArgsArray {
    PipeArgs a[kMaxRanks];
};

// Bytes of one ring slot.
HCCLB_HD uint64_t pipe_slot_bytes(int mode, uint64_t chunk_elems, int es, int p)
{
    const uint64_t c = chunk_elems * (uint64_t)es;
    switch (mode) {
        case PM_AR2_PUSH: case PM_RD_PUSH: return 2 * c;  // the p pushed slices, then the p reduced slices
        case PM_AR1_PUSH: case PM_RS_MC: case PM_RS_PUSH: return (uint64_t)p * c;
        default: return c;
    }
}
HCCLB_HD bool pipe_mode_is_mc(int mode) { return mode == PM_AR2_MC || mode == PM_AR1_MC || mode == PM_RS_MC || mode == PM_BC_MC; }
HCCLB_HD bool pipe_mode_is_bcast(int mode) { return mode == PM_BC_MC || mode == PM_BC_PUSH; }
HCCLB_HD bool pipe_mode_has_copy_out(int mode) { return mode == PM_AR2_MC || mode == PM_AR2_PUSH || mode == PM_RD_PUSH; }
HCCLB_HD bool pipe_mode_is_zc(int mode) { return mode == PM_AR1_ZC || mode == PM_RS_ZC || mode == PM_AG_ZC; }

// One launch runs the listed local ranks (more than one: virtual ranks of one GPU).  Always a cooperative launch: the
// stages of a rank wait on one another, so all CTAs have to be resident together.
HcclResult launch_pipe_coll(const RankCtx *dev_ctx, const PipeArgs *args, int nlocal, int redop, void *stream);

}  // namespace hcclb
