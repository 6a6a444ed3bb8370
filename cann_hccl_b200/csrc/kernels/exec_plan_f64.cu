// Plan executor and pipelined large-message kernels for element type double (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(double, f64)
HCCLB_INSTANTIATE_PIPE(double, f64)
}  // namespace hcclb
