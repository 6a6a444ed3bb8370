// Plan executor and pipelined large-message kernels for element type unsigned long long (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(unsigned long long, u64)
HCCLB_INSTANTIATE_PIPE(unsigned long long, u64)
}  // namespace hcclb
