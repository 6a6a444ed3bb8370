// Calibration of the selector on the communicator itself.  Two parts, both agreed over all ranks through the hub so that
// every rank selects with identical numbers:
//   1. the cost model's constants: launch overhead, flag-hop latency (alpha), peer bandwidth (beta), in-switch bandwidth and
//      local copy throughput (gamma), the bandwidths taken on messages of 32 MiB and more;
//   2. a measured table per collective (AllReduce, AllGather, ReduceScatter, Broadcast, Reduce, Scatter, Gather): every
//      candidate algorithm at a ladder of sizes.  Where a table exists the selector takes the fastest measured algorithm that is legal for the
//      (type, operator, determinism) at hand, and falls back on the model elsewhere.
// Runs once when a device communicator with more than one rank is created (HCCL_CALIBRATE=0 skips it; HcclB200Calibrate
// repeats it on demand).  The reference selects every op from one cost model with a fixed 60 us step latency
// (algorithm/impl/operator/coll_alg_operator.cc:32, :313-456) and no measurement.
#include <cuda_runtime.h>
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>
#include "common/log.h"
#include "core/communicator.h"
#include "kernels/ar_ll.h"

namespace hcclb {

namespace {
struct Timer {
    cudaEvent_t a, b;
    cudaStream_t s;
    explicit Timer(cudaStream_t st) : s(st) { cudaEventCreate(&a); cudaEventCreate(&b); }
    ~Timer() { cudaEventDestroy(a); cudaEventDestroy(b); }
    template <class F> double us(int warm, int iters, F &&f)
    {
        for (int i = 0; i < warm; ++i) f();
        cudaEventRecord(a, s);
        for (int i = 0; i < iters; ++i) f();
        cudaEventRecord(b, s);
        cudaEventSynchronize(b);
        float ms = 0;
        cudaEventElapsedTime(&ms, a, b);
        return ms * 1e3 / iters;
    }
};

struct Candidate {
    int coll;
    std::vector<int> algos;
};
}  // namespace

HcclResult Communicator::calibrate(void *stream)
{
    if (settings_.transport != TR_DEVICE || nranks_ < 2) return HCCL_SUCCESS;  // the host transport keeps the default model
    const int nl = nlocal(), p = nranks_;
    const EnvConfig &env = env_config();
    cudaStream_t st = (cudaStream_t)stream;
    bool own_stream = false;
    if (!st) {
        CHK_RET_LOG(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess, HCCL_E_RUNTIME, "cudaStreamCreate failed");
        own_stream = true;
    }
    // calibration traffic is not the application's: statistics, the op index (fault hooks count it) and the trace start
    // again afterwards; parameter checks over the hub are skipped (every rank runs this same code)
    const CommStats stats0 = stats_;
    const uint64_t op_index0 = op_index_;
    calibrating_ = true;
    struct Restore {
        Communicator *c; const CommStats &s; uint64_t oi; cudaStream_t st; bool own;
        ~Restore() { c->stats_ = s; c->op_index_ = oi; c->calibrating_ = false; if (own) cudaStreamDestroy(st); }
    } restore{this, stats0, op_index0, st, own_stream};

    // largest message per rank: 256 MiB for AllReduce / Broadcast / Reduce, half of that per rank for the collectives whose
    // other buffer is p times as large; virtual ranks of one GPU and small staging buffers scale it down
    uint64_t cap_mb = env.calibrate_max_mb > 0 ? (uint64_t)env.calibrate_max_mb : 256;
    if (all_local_) cap_mb = std::min<uint64_t>(cap_mb, 4);
    const uint64_t max_ar = std::max<uint64_t>(64u << 10, std::min<uint64_t>(cap_mb << 20, settings_.stage_half_bytes * 4));
    const uint64_t max_blk = std::max<uint64_t>(64u << 10, max_ar / 2);
    const size_t small_bytes = (size_t)max_ar, big_bytes = (size_t)max_blk * p;
    std::vector<void *> small(nl), big(nl);
    bool okalloc = true;
    for (int li = 0; li < nl; ++li) {
        small[li] = big[li] = nullptr;
        okalloc = okalloc && cudaMalloc(&small[li], small_bytes * 2) == cudaSuccess && cudaMalloc(&big[li], big_bytes) == cudaSuccess;
    }
    auto free_all = [&] {
        for (int li = 0; li < nl; ++li) { if (small[li]) cudaFree(small[li]); if (big[li]) cudaFree(big[li]); }
    };
    if (!okalloc) { free_all(); cudaGetLastError(); HLOG_WARN("calibration skipped: no memory for its buffers"); return HCCL_SUCCESS; }
    for (int li = 0; li < nl; ++li) { cudaMemsetAsync(small[li], 0, small_bytes * 2, st); cudaMemsetAsync(big[li], 0, big_bytes, st); }

    Timer t(st);
    HcclResult rc = HCCL_SUCCESS;
    // one collective on the calibration buffers; successive calls of small messages walk through disjoint windows, as an
    // application's tensors would (a table measured on one L2-resident buffer favours the algorithms that re-read most)
    uint64_t call = 0;
    std::vector<const void *> in(nl);
    std::vector<void *> out(nl);
    auto run = [&](int coll, int algo, uint64_t bytes, int nchan) {
        OpRequest rq;
        rq.coll = coll; rq.algo = algo; rq.count = bytes / 4; rq.dtype = HCCL_DATA_TYPE_FP32; rq.redop = HCCL_REDUCE_SUM; rq.nchan = nchan;
        rq.root = 0; rq.stream = st;
        const uint64_t nwin = std::max<uint64_t>(1, std::min<uint64_t>(8, bytes ? small_bytes / bytes : 1));
        const size_t off = (size_t)((call++ % nwin) * bytes);
        for (int li = 0; li < nl; ++li) {
            uint8_t *s0 = (uint8_t *)small[li], *b0 = (uint8_t *)big[li];
            switch (coll) {
                case COLL_ALLGATHER: case COLL_GATHER: in[li] = s0 + off; out[li] = b0; break;          // small -> big
                case COLL_REDUCE_SCATTER: case COLL_SCATTER: in[li] = b0; out[li] = s0 + off; break;    // big -> small
                case COLL_BROADCAST: in[li] = s0 + off; out[li] = s0 + off; break;           // in place, as the API has it
                default: in[li] = s0 + off; out[li] = s0 + small_bytes + off; break;         // AllReduce, Barrier
            }
        }
        rq.in = in.data(); rq.out = out.data();
        HcclResult r = collective(rq);
        if (r != HCCL_SUCCESS && rc == HCCL_SUCCESS) rc = r;
    };

    // ---- constants of the model
    const int nch = all_local_ ? std::max(1, 64 / p) : 32;
    const uint64_t bw_bytes = std::min<uint64_t>(max_blk, 32u << 20);
    double t_barrier = t.us(3, 20, [&] { run(COLL_BARRIER, ALGO_AUTO, 0, 1); });
    double t_small = t.us(3, 20, [&] { run(COLL_ALLREDUCE, ALGO_MESH_ONESHOT, 1024, 1); });
    double t_ag = t.us(2, 4, [&] { run(COLL_ALLGATHER, ALGO_MESH, bw_bytes, nch); });
    double t_nvls = nvls_ ? t.us(2, 4, [&] { run(COLL_ALLREDUCE, ALGO_NVLS, bw_bytes, nch); }) : 0;
    double t_copy = t.us(2, 4, [&] { cudaMemcpyAsync((uint8_t *)small[0] + small_bytes, small[0], bw_bytes, cudaMemcpyDeviceToDevice, st); });
    if (rc != HCCL_SUCCESS) { free_all(); return rc; }
    double vals[5];
    vals[0] = std::max(0.3, std::min(t_barrier * 0.5, t_small * 0.5));                                   // alpha
    vals[1] = std::max(0.5, t_barrier - vals[0]);                                                         // launch
    vals[2] = (double)(p - 1) * bw_bytes / std::max(1.0, t_ag - t_barrier) / 1e3;                        // beta GB/s: (p-1)n pulled per rank
    vals[3] = nvls_ && t_nvls > t_barrier ? (1.0 + 1.0 / p) * bw_bytes / (t_nvls - t_barrier) / 1e3 : 0;  // in-switch GB/s
    vals[4] = (double)bw_bytes / std::max(0.5, t_copy) / 1e3;                                             // gamma GB/s
    std::vector<std::string> all;
    CHK_RET(exchange("calib/" + std::to_string(seq_), std::string((const char *)vals, sizeof(vals)), &all));
    double avg[5] = {0, 0, 0, 0, 0};
    for (auto &s : all) {
        double v[5];
        memcpy(v, s.data(), sizeof(v));
        for (int i = 0; i < 5; ++i) avg[i] += v[i] / all.size();
    }
    model_.alpha_us = avg[0];
    model_.launch_us = avg[1];
    model_.beta_gbps = avg[2];
    if (avg[3] > 0) model_.nvls_gbps = avg[3];
    model_.gamma_gbps = avg[4];

    // ---- measured tables
    const std::vector<Candidate> cands = {
        {COLL_ALLREDUCE, {ALGO_LL, ALGO_MESH_ONESHOT, ALGO_NVLS_ONESHOT, ALGO_MESH, ALGO_NVLS, ALGO_RING, ALGO_MESH_PIPE, ALGO_NVLS_PIPE}},
        {COLL_ALLGATHER, {ALGO_LL, ALGO_MESH, ALGO_PAIRWISE, ALGO_RING, ALGO_NVLS, ALGO_MESH_PIPE}},
        {COLL_REDUCE_SCATTER, {ALGO_LL, ALGO_MESH, ALGO_RING, ALGO_NVLS, ALGO_MESH_PIPE, ALGO_NVLS_PIPE}},
        {COLL_BROADCAST, {ALGO_STAR, ALGO_RING, ALGO_TREE, ALGO_NVLS, ALGO_MESH_PIPE, ALGO_NVLS_PIPE}},
        {COLL_REDUCE, {ALGO_STAR, ALGO_RING, ALGO_TREE, ALGO_RHD, ALGO_MESH_PIPE}},
        {COLL_SCATTER, {ALGO_STAR, ALGO_RING}},
        {COLL_GATHER, {ALGO_STAR, ALGO_RING}},
    };
    std::vector<double> mine;
    std::vector<std::vector<uint64_t>> ladders;
    for (auto &cd : cands) {
        const bool blocked = cd.coll == COLL_ALLGATHER || cd.coll == COLL_REDUCE_SCATTER || cd.coll == COLL_SCATTER || cd.coll == COLL_GATHER;
        const uint64_t top = blocked ? max_blk : max_ar;
        std::vector<uint64_t> sizes;
        // steps of 4x, of 2x from 256 KiB on: that is where the algorithms cross over
        for (uint64_t sz = 16u << 10; sz <= top; sz *= (sz >= (256u << 10) ? 2 : 4)) sizes.push_back(sz);
        if (sizes.empty() || sizes.back() != top) sizes.push_back(top);
        ladders.push_back(sizes);
        for (uint64_t sz : sizes) {
            for (int a = 0; a < ALGO_COUNT; ++a) {
                double us = 0;
                const bool listed = std::find(cd.algos.begin(), cd.algos.end(), a) != cd.algos.end();
                const bool is_nvls = a == ALGO_NVLS || a == ALGO_NVLS_ONESHOT || a == ALGO_NVLS_PIPE;
                const bool is_pipe = a == ALGO_MESH_PIPE || a == ALGO_NVLS_PIPE;
                bool skip = !listed || (is_nvls && !nvls_);
                skip = skip || (a == ALGO_LL && (!ll_ok_ || sz > (cd.coll == COLL_ALLREDUCE ? ll_max_bytes() : ll_block_max())));
                skip = skip || (is_pipe && sz < (1u << 20));                                                   // three stages of hand-offs cost tens of microseconds
                skip = skip || ((a == ALGO_MESH_ONESHOT || a == ALGO_NVLS_ONESHOT) && sz > (8u << 20) && p > 2);  // (p-1) times the bytes
                skip = skip || ((a == ALGO_RING || a == ALGO_TREE) && sz < (256u << 10) && cd.coll != COLL_BROADCAST);
                if (!skip) {
                    const int iters = sz <= (1u << 20) ? 10 : (sz <= (16u << 20) ? 5 : 3);
                    us = t.us(2, iters, [&] { run(cd.coll, a, sz, 0); });
                }
                mine.push_back(us);
            }
        }
        if (rc != HCCL_SUCCESS) { free_all(); return rc; }
    }
    cudaStreamSynchronize(st);
    free_all();
    HcclResult src = async_error();
    if (src != HCCL_SUCCESS) return src;
    std::vector<std::string> allt;
    CHK_RET(exchange("tune/" + std::to_string(seq_), std::string((const char *)mine.data(), mine.size() * sizeof(double)), &allt));
    std::vector<double> mean(mine.size(), 0.0);
    for (auto &blob : allt) {
        if (blob.size() != mine.size() * sizeof(double)) { HLOG_ERROR("ranks measured different calibration ladders"); return HCCL_E_INTERNAL; }
        const double *v = (const double *)blob.data();
        for (size_t i = 0; i < mine.size(); ++i) mean[i] = std::max(mean[i], v[i]);  // an op is as slow as its slowest rank
    }
    tuned_.clear();
    size_t pos = 0;
    for (size_t ci = 0; ci < cands.size(); ++ci) {
        TunedTable tb;
        tb.sizes = ladders[ci];
        tb.us.assign(tb.sizes.size(), std::vector<double>(ALGO_COUNT, 0.0));
        for (size_t b = 0; b < tb.sizes.size(); ++b)
            for (int a = 0; a < ALGO_COUNT; ++a) tb.us[b][a] = mean[pos++];
        tuned_[cands[ci].coll] = std::move(tb);
    }
    HLOG_INFO("calibrated: alpha %.2f us, launch %.2f us, beta %.0f GB/s, nvls %.0f GB/s, gamma %.0f GB/s; tables for %zu collectives",
              model_.alpha_us, model_.launch_us, model_.beta_gbps, model_.nvls_gbps, model_.gamma_gbps, tuned_.size());
    return HCCL_SUCCESS;
}

}  // namespace hcclb
