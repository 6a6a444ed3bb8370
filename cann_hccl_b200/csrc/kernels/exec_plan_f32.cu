// Executor kernels for element type float (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(float, f32)
}  // namespace hcclb
