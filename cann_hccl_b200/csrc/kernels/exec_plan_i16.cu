// Plan executor and pipelined large-message kernels for element type int16_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(int16_t, i16)
HCCLB_INSTANTIATE_PIPE(int16_t, i16)
}  // namespace hcclb
