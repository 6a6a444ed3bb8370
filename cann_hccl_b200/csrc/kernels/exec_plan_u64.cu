// Executor kernels for element type unsigned long long (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(unsigned long long, u64)
}  // namespace hcclb
