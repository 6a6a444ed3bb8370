// Executor kernels for element type double (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(double, f64)
}  // namespace hcclb
