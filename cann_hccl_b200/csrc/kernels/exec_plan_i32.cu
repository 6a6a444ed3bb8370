// Plan executor and pipelined large-message kernels for element type int32_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(int32_t, i32)
HCCLB_INSTANTIATE_PIPE(int32_t, i32)
}  // namespace hcclb
