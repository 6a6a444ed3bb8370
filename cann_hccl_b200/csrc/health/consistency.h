// Parameter consistency between ranks and CRC32 (reference: common/health/rank_consistentcy_checker.{cc,h},
// calc_crc.cc — reflected polynomial 0xEDB88320).  Before the first use of an op shape every rank publishes its
// parameter frame through the hub; a mismatch fails the call with HCCL_E_PARA on every rank instead of letting
// kernels wait for data that never comes.  Disabled with HCCL_CONSISTENCY_CHECK=0.
#pragma once
#include <cstddef>
#include <cstdint>
namespace hcclb {
uint32_t crc32(const void *data, size_t len, uint32_t seed);
bool consistency_enabled();
struct OpFrame {
    int32_t coll, dtype, redop, root, algo, pad;
    uint64_t count;
    uint64_t stage_half;
    uint64_t zc_in, zc_out;  // (allocation << 48) ^ offset of the buffers of a zero-copy op, else 0
    uint32_t counts_crc, displs_crc;
};
}  // namespace hcclb
