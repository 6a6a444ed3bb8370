// Plan executor and pipelined large-message kernels for element type uint32_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(uint32_t, u32)
HCCLB_INSTANTIATE_PIPE(uint32_t, u32)
}  // namespace hcclb
