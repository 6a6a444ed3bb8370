// Algorithm selector: picks (algorithm, channel count) per collective from an alpha-beta-gamma cost model.
// Same closed forms as the reference's level-1 selector (algorithm/impl/operator/coll_alg_operator.cc:313-456:
// ring (p-1)a + (p-1)/p n/B, log-step ceil(log2 p)a + ..., non-power-of-two RHD (2p-1)/p) extended with
// mesh one-shot / two-shot and in-switch (NVLS) terms.  alpha/beta/gamma are measured per communicator by the
// calibration pass instead of the reference's fixed 60 us; every rank uses the same agreed numbers so that all
// ranks select the same algorithm.  Ties break in a fixed order (mesh > ring > rhd), like the reference's
// Ring > NHR > HD order.
#pragma once
#include <string>
#include "algo/schedule.h"
#include "common/env.h"
namespace hcclb {

struct CostModel {
    double alpha_us = 1.8;     // one flag hop between two GPUs (signal store -> visible to a polling peer)
    double launch_us = 2.5;    // fixed cost of the kernel itself (launch + first/last CTA bookkeeping)
    double beta_gbps = 650.0;  // achievable P2P load/store bandwidth per direction per GPU
    double nvls_gbps = 800.0;  // achievable multimem bandwidth per GPU
    double gamma_gbps = 2500.0;  // local HBM copy/reduce throughput (read+write counted once)
    double step_us = 0.6;      // per-step overhead inside the executor (barrier + flag bookkeeping)
};

struct SelectInput {
    int coll = COLL_ALLREDUCE;
    uint64_t bytes = 0;  // message bytes per rank in the sense of the API count (AllGather: sendCount bytes, ...)
    int nranks = 1;
    int dtype = HCCL_DATA_TYPE_FP32;
    int redop = HCCL_REDUCE_SUM;
    bool deterministic = false;
    bool nvls = false;          // multicast mapping available
    bool device = true;         // false: host transport (NVLS never applies)
    int expansion_mode = 0;     // 1 = host-orchestrated: plain algorithms only
    int max_channels = 32;
    uint64_t ll_max_bytes = 0;  // largest message the LL kernel may take (0 = LL unavailable)
    std::string forced;         // algorithm name from HCCL_ALGO for this collective ("" = none)
};
struct Selection {
    int algo = ALGO_MESH;
    int nchan = 1;
    double est_us = 0;
};

// Modelled time of one (collective, algorithm) pair; < 0 when the pair does not exist.
double estimate_us(int coll, int algo, uint64_t bytes, int p, const CostModel &m);
// True when multimem.ld_reduce supports this (dtype, op) pair and the byte count is a multiple of 16.
bool nvls_reduce_supported(int dtype, int redop, uint64_t bytes);
Selection select_algo(const SelectInput &in, const CostModel &m);
// Channel (CTA) count for a message of `bytes` per rank.
int pick_channels(uint64_t bytes, int max_channels);
// HCCL_ALGO key of a collective ("allreduce", ...).
const char *coll_env_key(int coll);
std::string forced_algo_for(const EnvConfig &env, int coll);

}  // namespace hcclb
