// Executor kernels for element type long long (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(long long, i64)
}  // namespace hcclb
