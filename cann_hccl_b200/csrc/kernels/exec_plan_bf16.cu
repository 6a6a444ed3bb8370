// Plan executor and pipelined large-message kernels for element type __nv_bfloat16 (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(__nv_bfloat16, bf16)
HCCLB_INSTANTIATE_PIPE(__nv_bfloat16, bf16)
}  // namespace hcclb
