// Address resolution shared by the device executor kernel and the host executor.
#pragma once
#include "algo/plan.h"
namespace hcclb {
// Address of byte `off` of buffer `buf` owned by `rank` as seen from the executing rank.
// RANK_ALL on the staging buffer selects the NVLS multicast mapping.
HCCLB_HD uint8_t *resolve_addr(const RankCtx &c, const ExecArgs &a, uint8_t buf, int rank, uint64_t off, uint64_t half_off)
{
    switch (buf) {
        case BUF_IN: return const_cast<uint8_t *>(a.in) + off;
        case BUF_OUT: return a.out + off;
        case BUF_STAGE:
            if (rank == RANK_ALL) return c.mc_stage + half_off + off;
            return c.stage[rank == RANK_SELF ? c.rank : rank] + half_off + off;
        case BUF_P2P: return c.p2p[rank == RANK_SELF ? c.rank : rank] + off;
        case BUF_ZIN:
            if (rank == RANK_SELF) return const_cast<uint8_t *>(a.in) + off;
            return (rank == RANK_ALL ? a.z_in_mc : a.z_in_peer[rank] + a.z_in_off) + off;
        case BUF_ZOUT:
            if (rank == RANK_SELF) return a.out + off;
            return (rank == RANK_ALL ? a.z_out_mc : a.z_out_peer[rank] + a.z_out_off) + off;
        default: return nullptr;
    }
}
HCCLB_HD uint64_t flag_value(const ExecArgs &a, const Step &s, uint32_t val)
{
    return (s.flags & SF_ABS_VALS) ? (uint64_t)val : ((a.seq << kSeqShift) + val);
}
}  // namespace hcclb
