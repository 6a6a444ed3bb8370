// Launch interface of the Inf / NaN scan (kernels/overflow.cu).
#pragma once
#include <cstdint>
#include "hccl/hccl_types.h"
namespace hcclb {
// Adds the number of non-finite elements of buf[0, count) to *counter (host-mapped memory), stream-ordered.
HcclResult launch_overflow_scan(const void *buf, uint64_t count, int dtype, unsigned long long *counter, void *stream);
}  // namespace hcclb
