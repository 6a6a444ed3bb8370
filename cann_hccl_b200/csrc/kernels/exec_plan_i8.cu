// Executor kernels for element type int8_t (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(int8_t, i8)
}  // namespace hcclb
