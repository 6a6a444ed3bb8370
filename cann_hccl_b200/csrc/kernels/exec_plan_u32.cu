// Executor kernels for element type uint32_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(uint32_t, u32)
}  // namespace hcclb
