// Launch interface of the low-latency small-message AllReduce kernel (kernels/ar_ll.cu).
#pragma once
#include "algo/plan.h"
namespace hcclb {
constexpr int kLlThreads = 256;
constexpr uint64_t kLlMaxPayload = 2u << 20;          // largest message the LL path takes (bytes); mailboxes cost 4 x ranks x this per rank
constexpr uint64_t kLlSlotBytes = 2 * kLlMaxPayload;  // 16-byte lines carry 8 payload bytes
// Largest message of the two-shot form: its two areas of p pieces share the mailbox half of p slots, a piece carries 1/p of
// the message at 50 % payload.
HCCLB_HD uint64_t ll_two_shot_max(int p) { return (uint64_t)p * kLlSlotBytes / 4 / 16 * 16; }
// Largest block (bytes per rank) of the LL ReduceScatter / AllGather: one piece of an area at 50 % payload.
HCCLB_HD uint64_t ll_block_max() { return kLlSlotBytes / 4 / 16 * 16; }
enum LlKind : uint32_t { LL_AR_ONESHOT = 0, LL_AR_TWOSHOT = 1, LL_REDUCE_SCATTER = 2, LL_ALLGATHER = 3 };
struct LlArgs {
    uint8_t *ll[kMaxRanks];   // mailbox region of rank q mapped into this rank's address space
    const void *in;
    void *out;
    uint64_t count;           // elements
    uint64_t slot_bytes;
    uint64_t timeout_ns;
    uint64_t seq;
    DevStatus *status;
    volatile uint32_t *abort;
    uint32_t *local_fail;
    uint32_t *exit_counter;   // device counter that finds the last CTA of the op
    uint64_t *dev_tail;       // device word of the op-execution counter: set to `exe_id` when the op has completed
    uint64_t exe_id;          // value the host wrote into the status block's head when it launched the op
    int32_t rank, nranks;
    uint32_t tag, parity;
    uint32_t two_shot, pad;   // LlKind: 1 = slices go to their owners, reduced slices come back; 2 / 3 = the two halves of that as
                              // ReduceScatter and AllGather (count = elements of one rank's block)
};
struct LlArgsArray {
    LlArgs a[kMaxRanks];
};
// One launch runs the listed local ranks (more than one: virtual ranks of one GPU, cooperative launch).
HcclResult launch_ar_ll(const LlArgs *args, int nlocal, int dtype, int op, void *stream);
}  // namespace hcclb
