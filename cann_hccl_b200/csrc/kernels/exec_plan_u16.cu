// Plan executor and pipelined large-message kernels for element type uint16_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(uint16_t, u16)
HCCLB_INSTANTIATE_PIPE(uint16_t, u16)
}  // namespace hcclb
