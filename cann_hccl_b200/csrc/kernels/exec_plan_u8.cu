// Plan executor and pipelined large-message kernels for element type uint8_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(uint8_t, u8)
HCCLB_INSTANTIATE_PIPE(uint8_t, u8)
}  // namespace hcclb
