// Host-memory transport: interprets a Plan on a CPU rank (thread or process).  Peers' staging and flag
// pages are ordinary shared memory; flags use acquire/release atomics.  It is the correctness oracle for
// every schedule and the transport of HCCL_TRANSPORT=host communicators.
#pragma once
#include "algo/plan.h"
namespace hcclb {
// Runs the steps of one rank to completion (or until a wait times out / the abort word is raised).
// Returns HCCL_SUCCESS, HCCL_E_TIMEOUT or HCCL_E_SUSPENDING; the status block of `c` is filled on failure.
HcclResult exec_plan_host(const RankCtx &c, const ExecArgs &a);
}  // namespace hcclb
