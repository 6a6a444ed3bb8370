// Plan executor and pipelined large-message kernels for element type __half (all four reduction operators).
#include "kernels/exec_plan_impl.cuh"
#include "kernels/pipe_coll.cuh"
namespace hcclb {
HCCLB_INSTANTIATE_EXEC(__half, f16)
HCCLB_INSTANTIATE_PIPE(__half, f16)
}  // namespace hcclb
