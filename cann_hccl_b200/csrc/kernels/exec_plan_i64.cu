// Plan executor and pipelined large-message kernels for element type long long (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(long long, i64)
HCCLB_INSTANTIATE_PIPE(long long, i64)
}  // namespace hcclb
