// Plan executor and pipelined large-message kernels for element type int8_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(int8_t, i8)
HCCLB_INSTANTIATE_PIPE(int8_t, i8)
}  // namespace hcclb
