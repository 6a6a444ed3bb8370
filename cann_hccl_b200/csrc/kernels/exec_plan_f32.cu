// Plan executor and pipelined large-message kernels for element type float (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(float, f32)
HCCLB_INSTANTIATE_PIPE(float, f32)
}  // namespace hcclb
