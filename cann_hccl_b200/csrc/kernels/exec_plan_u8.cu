// Executor kernels for element type uint8_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(uint8_t, u8)
}  // namespace hcclb
