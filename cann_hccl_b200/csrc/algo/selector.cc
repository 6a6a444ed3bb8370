#include "algo/selector.h"
#include <algorithm>
#include <cmath>

namespace hcclb {

const char *coll_env_key(int coll)
{
    switch (coll) {
        case COLL_ALLREDUCE: return "allreduce";
        case COLL_BROADCAST: return "broadcast";
        case COLL_REDUCE_SCATTER: case COLL_REDUCE_SCATTER_V: return "reducescatter";
        case COLL_SCATTER: return "scatter";
        case COLL_ALLGATHER: case COLL_ALLGATHER_V: return "allgather";
        case COLL_ALLTOALL: case COLL_ALLTOALLV: case COLL_ALLTOALLVC: return "alltoall";
        case COLL_REDUCE: return "reduce";
        case COLL_GATHER: return "gather";
        default: return "other";
    }
}
std::string forced_algo_for(const EnvConfig &env, int coll)
{
    auto it = env.algo.find(coll_env_key(coll));
    if (it != env.algo.end()) return it->second;
    it = env.algo.find("*");
    return it != env.algo.end() ? it->second : std::string();
}

bool nvls_reduce_supported(int dtype, int redop, uint64_t bytes)
{
    if (bytes % 16 != 0) return false;
    bool minmax = redop == HCCL_REDUCE_MAX || redop == HCCL_REDUCE_MIN;
    if (redop != HCCL_REDUCE_SUM && !minmax) return false;  // no in-switch product
    switch (dtype) {
        case HCCL_DATA_TYPE_FP32: return redop == HCCL_REDUCE_SUM;  // multimem has no f32 min/max
        case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_BFP16: return true;
        case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_UINT32: return true;
        default: return false;
    }
}

static bool algo_exists(int coll, int algo)
{
    switch (coll) {
        case COLL_ALLREDUCE: return algo == ALGO_MESH || algo == ALGO_MESH_ONESHOT || algo == ALGO_RING || algo == ALGO_RHD || algo == ALGO_NVLS || algo == ALGO_NVLS_ONESHOT || algo == ALGO_MESH_PIPE || algo == ALGO_NVLS_PIPE || algo == ALGO_LL || algo == ALGO_NVLS_ZC;
        case COLL_REDUCE_SCATTER: return algo == ALGO_MESH || algo == ALGO_RING || algo == ALGO_RHD || algo == ALGO_NVLS || algo == ALGO_MESH_PIPE || algo == ALGO_NVLS_PIPE || algo == ALGO_LL;
        case COLL_ALLGATHER: return algo == ALGO_MESH || algo == ALGO_RING || algo == ALGO_RHD || algo == ALGO_NVLS || algo == ALGO_PAIRWISE || algo == ALGO_MESH_PIPE || algo == ALGO_LL;
        case COLL_REDUCE_SCATTER_V: return algo == ALGO_MESH || algo == ALGO_RING || algo == ALGO_NVLS;
        case COLL_ALLGATHER_V: return algo == ALGO_MESH || algo == ALGO_RING || algo == ALGO_NVLS || algo == ALGO_PAIRWISE;
        case COLL_BROADCAST: return algo == ALGO_STAR || algo == ALGO_RING || algo == ALGO_TREE || algo == ALGO_NVLS || algo == ALGO_MESH_PIPE || algo == ALGO_NVLS_PIPE;
        case COLL_REDUCE: return algo == ALGO_STAR || algo == ALGO_RING || algo == ALGO_TREE || algo == ALGO_RHD || algo == ALGO_MESH_PIPE;
        case COLL_SCATTER: case COLL_GATHER: return algo == ALGO_STAR || algo == ALGO_RING;
        case COLL_ALLTOALL: case COLL_ALLTOALLV: case COLL_ALLTOALLVC: return algo == ALGO_MESH || algo == ALGO_PAIRWISE;
        default: return false;
    }
}

double estimate_us(int coll, int algo, uint64_t bytes, int p, const CostModel &m)
{
    if (!algo_exists(coll, algo) || p < 2) return -1;
    const double n = (double)bytes, B = m.beta_gbps * 1e3, Bn = m.nvls_gbps * 1e3, G = m.gamma_gbps * 1e3;  // bytes per us
    const double a = m.alpha_us, L = m.launch_us, s = m.step_us;
    const double lg = std::ceil(std::log2((double)p));
    const bool pow2 = (p & (p - 1)) == 0;
    const double f = (double)(p - 1) / p;
    // link bytes per chunk of the pipelined kernels (Communicator::run_pipe): 1/16 of what crosses the links, 4 to 8 MiB
    const double fan = (coll == COLL_REDUCE_SCATTER || coll == COLL_ALLGATHER) ? p : 1.0;
    const double chunk = std::min(n * fan, std::min(8.0 * (1 << 20), std::max(4.0 * (1 << 20), n * fan / 16)));
    switch (coll) {
        case COLL_ALLREDUCE:
            switch (algo) {
                case ALGO_NVLS_ZC: return L + 2 * a + (1.0 + 1.0 / p) * n / Bn + 3 * s;
                case ALGO_LL: return L + 0.6 * a + 2.0 * (p - 1) * n / B + 2.0 * p * n / G;  // lines carry 50 % payload; no fence, no flag hop
                case ALGO_MESH_ONESHOT: return L + a + (p - 1) * n / B + n / G + 2 * s;
                case ALGO_MESH: return L + 2 * a + 2 * f * n / B + 2 * n / G + (p + 2) * s;
                case ALGO_RING: return L + 2 * (p - 1) * (a + s) + 2 * f * n / B + n / G;
                case ALGO_RHD: return L + (2 * lg + (pow2 ? 0 : 2)) * (a + s) + (pow2 ? 2 * f : 2.0 * (2 * p - 1) / p) * n / B + n / G;
                case ALGO_NVLS_ONESHOT: return L + a + p * n / Bn + n / G + 2 * s;
                case ALGO_NVLS: return L + 2 * a + (1.0 + 1.0 / p) * n / Bn + 2 * n / G + (p + 2) * s;
                // pipelined kernels: the local copies hide behind the transfer; the price is a pipeline fill of one chunk per stage
                case ALGO_MESH_PIPE: return L + (p == 2 ? 2 : 3) * a + (p == 2 ? 1.0 : 2 * f) * n / B + 3 * chunk / B;
                case ALGO_NVLS_PIPE: return L + (p == 2 ? 2 : 3) * a + (p == 2 ? 1.0 : 1.0 + 1.0 / p) * n / Bn + 3 * chunk / Bn;
            }
            break;
        case COLL_REDUCE_SCATTER: case COLL_REDUCE_SCATTER_V:  // bytes = one rank's result
            switch (algo) {
                case ALGO_LL: return L + 0.6 * a + 2.0 * (p - 1) * n / B + p * n / G;  // lines carry 50 % payload; no fence, no flag hop
                case ALGO_MESH: return L + a + (p - 1) * n / B + p * n / G + (p + 1) * s;
                case ALGO_RING: return L + (p - 1) * (a + s) + (p - 1) * n / B;
                case ALGO_RHD: return L + (lg + (pow2 ? 0 : 1)) * (a + s) + (pow2 ? (p - 1) : (2 * p - 1)) * n / B + p * n / G;
                case ALGO_NVLS: return L + a + n * (double)p / Bn / p * (p - 1) + p * n / G + (p + 1) * s;
                case ALGO_MESH_PIPE: return L + 2 * a + (p - 1) * n / B + 2 * chunk / B;
                case ALGO_NVLS_PIPE: return L + 2 * a + (p - 1) * n / Bn + 2 * chunk / Bn;
            }
            break;
        case COLL_ALLGATHER: case COLL_ALLGATHER_V:  // bytes = one rank's contribution
            switch (algo) {
                case ALGO_LL: return L + 0.6 * a + 2.0 * (p - 1) * n / B + p * n / G;
                case ALGO_MESH: return L + a + (p - 1) * n / B + n / G + 2 * s;
                case ALGO_RING: return L + (p - 1) * (a + s) + (p - 1) * n / B;
                case ALGO_PAIRWISE: return L + a + (p - 1) * n / B + (p - 1) * n / G + (p + 1) * s;  // push: no staging copy, copy-out per slot
                case ALGO_RHD: return L + (lg + (pow2 ? 0 : 2)) * (a + s) + (pow2 ? (p - 1) : (2 * p - 1)) * n / B;
                case ALGO_NVLS: return L + a + (p - 1) * n / Bn + p * n / G + 2 * s;
                case ALGO_MESH_PIPE: return L + 2 * a + (p - 1) * n / B + 2 * chunk / B;
            }
            break;
        case COLL_BROADCAST:
            switch (algo) {
                case ALGO_STAR: return L + a + n / G + (p - 1) * n / B + 2 * s;  // every non-root pulls n from the root: root egress (p-1)n
                case ALGO_RING: return L + (p - 1 + 3) * (a + s) + (1.0 + (p - 2) / 4.0) * n / B;
                case ALGO_TREE: return L + lg * (a + s) + lg * n / B;
                case ALGO_NVLS: return L + a + n / Bn + n / G;
                case ALGO_MESH_PIPE: return L + n / B + (p - 1) * (a + chunk / B);  // chain: every hop adds one chunk
                case ALGO_NVLS_PIPE: return L + 2 * a + n / Bn + 2 * chunk / Bn;
            }
            break;
        case COLL_REDUCE:
            switch (algo) {
                case ALGO_STAR: return L + a + (p - 1) * n / B + n / G;
                case ALGO_RING: return L + (p - 1 + 3) * (a + s) + (1.0 + (p - 2) / 4.0) * n / B;
                case ALGO_TREE: return L + lg * (a + s) + lg * n / B;
                case ALGO_RHD: return L + (lg + 1 + (pow2 ? 0 : 1)) * (a + s) + 2 * f * n / B;
                case ALGO_MESH_PIPE: return L + 3 * a + 2 * f * n / B + 3 * chunk / B;  // the root takes in p-1 pushed and p-1 reduced slices
            }
            break;
        case COLL_SCATTER: case COLL_GATHER:
            switch (algo) {
                case ALGO_STAR: return L + a + (p - 1) * n / B + p * n / G;
                case ALGO_RING: return L + (p - 1) * (a + s) + (p - 1) * p / 2.0 * n / B;
            }
            break;
        case COLL_ALLTOALL: case COLL_ALLTOALLV: case COLL_ALLTOALLVC:  // bytes = everything one rank sends
            switch (algo) {
                case ALGO_MESH: return L + a + f * n / B + n / G + 2 * s;
                case ALGO_PAIRWISE: return L + a + (p - 1) * s + f * n / B + n / G;
            }
            break;
    }
    return -1;
}

int pick_channels(uint64_t bytes, int max_channels)
{
    // one CTA per 16 KiB: a CTA keeps about 64 KB of loads in flight, so small messages finish in one round trip per
    // phase while large ones spread over enough CTAs to fill the links
    uint64_t c = bytes / (16u << 10);
    if (c < 1) c = 1;
    if (c > (uint64_t)max_channels) c = (uint64_t)max_channels;
    return (int)c;
}

Selection select_algo(const SelectInput &in, const CostModel &m)
{
    Selection sel;
    sel.nchan = pick_channels(in.bytes, in.max_channels);
    if (in.nranks <= 1) {
        sel.algo = ALGO_SINGLE;
        return sel;
    }
    bool reducing = in.coll == COLL_ALLREDUCE || in.coll == COLL_REDUCE_SCATTER || in.coll == COLL_REDUCE_SCATTER_V || in.coll == COLL_REDUCE;
    uint64_t nvls_bytes = in.bytes;
    if (in.coll == COLL_ALLREDUCE) nvls_bytes = in.bytes;  // slices are rounded to 16 bytes by the generator
    bool nvls_ok = in.nvls && in.device && !in.deterministic && in.expansion_mode != 1 &&
                   (reducing ? nvls_reduce_supported(in.dtype, in.redop, nvls_bytes) : in.bytes % 16 == 0);
    auto allowed = [&](int algo) {
        if (!algo_exists(in.coll, algo)) return false;
        if (algo == ALGO_NVLS || algo == ALGO_NVLS_ONESHOT || algo == ALGO_NVLS_PIPE) return nvls_ok;
        if (algo == ALGO_NVLS_ZC) return false;  // chosen by the communicator when the buffers are registered, never by the model
        if (algo == ALGO_LL) return in.device && in.expansion_mode != 1 && in.ll_max_bytes > 0 && in.bytes <= in.ll_max_bytes;
        if ((algo == ALGO_MESH_PIPE || algo == ALGO_NVLS_PIPE) && (!in.device || in.expansion_mode == 1)) return false;  // device kernels only
        return true;
    };
    if (!in.forced.empty()) {
        int a = algo_from_name(in.forced);
        // rooted and alltoall collectives accept the generic names of their families
        if (a == ALGO_MESH && !algo_exists(in.coll, ALGO_MESH) && algo_exists(in.coll, ALGO_STAR)) a = ALGO_STAR;
        if (a == ALGO_STAR && !algo_exists(in.coll, ALGO_STAR) && algo_exists(in.coll, ALGO_MESH)) a = ALGO_MESH;
        if (a == ALGO_RHD && !algo_exists(in.coll, ALGO_RHD) && algo_exists(in.coll, ALGO_TREE)) a = ALGO_TREE;
        if (a != ALGO_AUTO && allowed(a)) {
            sel.algo = a;
            sel.est_us = estimate_us(in.coll, a, in.bytes, in.nranks, m);
            return sel;
        }
    }
    static const int order[] = {ALGO_LL, ALGO_MESH_ONESHOT, ALGO_MESH, ALGO_STAR, ALGO_NVLS_ONESHOT, ALGO_NVLS, ALGO_MESH_PIPE, ALGO_NVLS_PIPE, ALGO_PAIRWISE, ALGO_RING, ALGO_TREE, ALGO_RHD};
    double best = -1;
    for (int a : order) {
        if (!allowed(a)) continue;
        double t = estimate_us(in.coll, a, in.bytes, in.nranks, m);
        if (t < 0) continue;
        if (best < 0 || t < best * (1.0 - 1e-9)) {
            best = t;
            sel.algo = a;
        }
    }
    sel.est_us = best;
    return sel;
}

}  // namespace hcclb
