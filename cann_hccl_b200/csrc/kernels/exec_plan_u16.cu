// Executor kernels for element type uint16_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(uint16_t, u16)
}  // namespace hcclb
