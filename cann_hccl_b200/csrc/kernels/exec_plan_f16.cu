// Executor kernels for element type __half (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(__half, f16)
}  // namespace hcclb
