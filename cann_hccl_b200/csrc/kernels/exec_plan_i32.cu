// Executor kernels for element type int32_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(int32_t, i32)
}  // namespace hcclb
