// Executor kernels for element type __nv_bfloat16 (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(__nv_bfloat16, bf16)
}  // namespace hcclb
