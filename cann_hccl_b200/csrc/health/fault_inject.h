// Host-side fault injection for tests (the reference has none).  HCCL_FAULT_INJECT is a ';'-separated list:
//   stall_rank:rank=R,op=N,ms=T[,attempts=K]  rank R sleeps T ms before executing its N-th collective (and before its
//                                   first K retries of that collective)
//   drop_heartbeat:rank=R[,after=N] rank R stops sending heartbeats (after N beats)
//   exit_rank:rank=R,op=N           rank R's process exits (code 17) instead of executing its N-th collective
// Faults are only ever produced on the host: no kernel is made to trap, hang or touch a bad address.
#pragma once
#include <cstdint>
namespace hcclb {
namespace fault {
void before_op(int rank, uint64_t op_index);
void before_attempt(int rank, uint64_t op_index, int attempt);  // attempt 1.. = retries of the op
bool drop_heartbeat(int rank);
void reload();  // re-read HCCL_FAULT_INJECT (tests)
}  // namespace fault
}  // namespace hcclb
