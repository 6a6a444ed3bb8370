// Calibration of the selector's cost model on the communicator itself: launch overhead, flag-hop latency (alpha),
// peer bandwidth (beta), in-switch bandwidth and local copy/reduce throughput (gamma) are timed with CUDA events
// and averaged over all ranks through the hub, so that every rank selects with identical numbers.
// (The reference's selector uses a fixed 60 us step latency, coll_alg_operator.cc:32.)
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
uint64_t si_ll_max() { return kLlMaxPayload; }
struct Timer {
    cudaEvent_t a, b;
    cudaStream_t s;
    explicit Timer(cudaStream_t st) : s(st) { cudaEventCreate(&a); cudaEventCreate(&b); }
    ~Timer() { cudaEventDestroy(a); cudaEventDestroy(b); }
    template <class F> double us(int iters, F &&f)
    {
        for (int i = 0; i < 3; ++i) f();
        cudaEventRecord(a, s);
        for (int i = 0; i < iters; ++i) f();
        cudaEventRecord(b, s);
        cudaEventSynchronize(b);
        float ms = 0;
        cudaEventElapsedTime(&ms, a, b);
        return ms * 1e3 / iters;
    }
};
}  // namespace

HcclResult Communicator::calibrate(void *stream)
{
    if (settings_.transport != TR_DEVICE) return HCCL_SUCCESS;  // the host transport keeps the default model
    if (nranks_ < 2) return HCCL_SUCCESS;
    cudaStream_t st = (cudaStream_t)stream;
    int nl = nlocal();
    size_t big = std::min<size_t>(settings_.stage_half_bytes / (size_t)nranks_ / 2, 16u << 20) / 256 * 256;
    if (big < 4096) return HCCL_E_MEMORY;
    std::vector<void *> in(nl), out(nl);
    for (int li = 0; li < nl; ++li) {
        CHK_RET_LOG(cudaMalloc(&in[li], big) != cudaSuccess || cudaMalloc(&out[li], big * nranks_) != cudaSuccess, HCCL_E_MEMORY, "calibration buffers");
        cudaMemsetAsync(in[li], 0, big, st);
    }
    Timer t(st);
    HcclResult rc = HCCL_SUCCESS;
    auto run = [&](int coll, int algo, uint64_t count, int nchan) {
        OpRequest rq;
        rq.coll = coll; rq.algo = algo; rq.count = count; rq.dtype = HCCL_DATA_TYPE_FP32; rq.redop = HCCL_REDUCE_SUM; rq.nchan = nchan;
        rq.in = (const void *const *)in.data(); rq.out = out.data(); rq.stream = stream;
        HcclResult r = collective(rq);
        if (r != HCCL_SUCCESS) rc = r;
    };
    double t_barrier = t.us(20, [&] { run(COLL_BARRIER, ALGO_AUTO, 0, 1); });
    double t_small = t.us(20, [&] { run(COLL_ALLREDUCE, ALGO_MESH_ONESHOT, 256, 1); });
    uint64_t cnt = big / 4;
    int nch = all_local_ ? std::max(1, 64 / nranks_) : 32;
    double t_ag = t.us(5, [&] { run(COLL_ALLGATHER, ALGO_MESH, cnt, nch); });
    double t_nvls = 0;
    if (nvls_) t_nvls = t.us(5, [&] { run(COLL_ALLREDUCE, ALGO_NVLS, cnt, nch); });
    for (int li = 0; li < nl; ++li) { cudaFree(in[li]); cudaFree(out[li]); }
    CHK_RET(rc);
    CHK_RET(sync_stream(stream));
    // model: barrier = launch + alpha; allgather(mesh) = launch + alpha + (p-1)n/B + n/G
    double vals[4];
    vals[0] = std::max(0.3, std::min(t_barrier * 0.5, t_small * 0.5));          // alpha
    vals[1] = std::max(0.5, t_barrier - vals[0]);                                // launch
    double xfer = std::max(1.0, t_ag - t_barrier);
    vals[2] = (double)(nranks_ - 1) * big / xfer / 1e3;                          // beta GB/s
    vals[3] = nvls_ && t_nvls > t_barrier ? (1.0 + 1.0 / nranks_) * big / (t_nvls - t_barrier) / 1e3 : 0;
    std::vector<std::string> all;
    CHK_RET(exchange("calib/" + std::to_string(seq_), std::string((const char *)vals, sizeof(vals)), &all));
    double avg[4] = {0, 0, 0, 0};
    for (auto &s : all) {
        double v[4];
        memcpy(v, s.data(), sizeof(v));
        for (int i = 0; i < 4; ++i) avg[i] += v[i] / all.size();
    }
    model_.alpha_us = avg[0];
    model_.launch_us = avg[1];
    model_.beta_gbps = avg[2];
    if (avg[3] > 0) model_.nvls_gbps = avg[3];
    // ---- measured AllReduce table: every candidate algorithm at a ladder of sizes, agreed over all ranks
    {
        static const int cands[] = {ALGO_LL, ALGO_MESH_ONESHOT, ALGO_NVLS_ONESHOT, ALGO_MESH, ALGO_NVLS, ALGO_RING, ALGO_MESH_PIPE, ALGO_NVLS_PIPE};
        std::vector<uint64_t> sizes;
        for (uint64_t sz = 16u << 10; sz <= (256u << 20) && sz <= settings_.stage_half_bytes / 2; sz *= 2) sizes.push_back(sz);
        size_t maxb = sizes.empty() ? 0 : sizes.back();
        std::vector<void *> tin(nl), tout(nl);
        bool okalloc = maxb > 0;
        for (int li = 0; li < nl && okalloc; ++li)
            okalloc = cudaMalloc(&tin[li], maxb) == cudaSuccess && cudaMalloc(&tout[li], maxb) == cudaSuccess;
        if (okalloc) {
            for (int li = 0; li < nl; ++li) cudaMemsetAsync(tin[li], 0, maxb, st);
            std::vector<double> mine(sizes.size() * ALGO_COUNT, 0.0);
            for (size_t b = 0; b < sizes.size(); ++b) {
                for (int algo : cands) {
                    bool is_nvls = algo == ALGO_NVLS || algo == ALGO_NVLS_ONESHOT || algo == ALGO_NVLS_PIPE;
                    if ((algo == ALGO_MESH_PIPE || algo == ALGO_NVLS_PIPE) && sizes[b] < (16u << 20)) continue;
                    if (is_nvls && !nvls_) continue;
                    if (algo == ALGO_LL && (!ll_ok_ || sizes[b] > si_ll_max())) continue;
                    // with two ranks one-shot moves no more bytes than two-shot and saves a phase: a candidate at every size
                    if ((algo == ALGO_MESH_ONESHOT || algo == ALGO_NVLS_ONESHOT) && sizes[b] > (8u << 20) && nranks_ > 2) continue;
                    if (algo == ALGO_RING && sizes[b] < (1u << 20)) continue;
                    int iters = sizes[b] <= (1u << 20) ? 12 : (sizes[b] <= (16u << 20) ? 6 : 3);
                    OpRequest rq;
                    rq.coll = COLL_ALLREDUCE; rq.algo = algo; rq.count = sizes[b] / 4; rq.dtype = HCCL_DATA_TYPE_FP32; rq.redop = HCCL_REDUCE_SUM;
                    rq.stream = stream;
                    // successive calls walk through disjoint windows of the buffers, as an application's tensors would: a
                    // table measured on one L2-resident buffer favours the algorithms that re-read their input most
                    const uint64_t nwin = std::max<uint64_t>(1, std::min<uint64_t>(8, maxb / sizes[b]));
                    uint64_t call = 0;
                    std::vector<const void *> win_in(nl);
                    std::vector<void *> win_out(nl);
                    mine[b * ALGO_COUNT + algo] = t.us(iters, [&] {
                        const size_t off = (size_t)((call++ % nwin) * sizes[b]);
                        for (int li = 0; li < nl; ++li) { win_in[li] = (const uint8_t *)tin[li] + off; win_out[li] = (uint8_t *)tout[li] + off; }
                        rq.in = win_in.data(); rq.out = win_out.data();
                        HcclResult r = collective(rq);
                        if (r != HCCL_SUCCESS) rc = r;
                    });
                }
            }
            for (int li = 0; li < nl; ++li) { cudaFree(tin[li]); cudaFree(tout[li]); }
            CHK_RET(rc);
            std::vector<std::string> allt;
            CHK_RET(exchange("tune/" + std::to_string(seq_), std::string((const char *)mine.data(), mine.size() * sizeof(double)), &allt));
            tuned_us_.assign(sizes.size(), std::vector<double>(ALGO_COUNT, 0.0));
            for (auto &sblob : allt) {
                const double *v = (const double *)sblob.data();
                for (size_t i = 0; i < mine.size(); ++i) tuned_us_[i / ALGO_COUNT][i % ALGO_COUNT] += v[i] / allt.size();
            }
            tuned_sizes_ = sizes;
        }
    }
    HLOG_INFO("calibrated: alpha %.2f us, launch %.2f us, beta %.0f GB/s, nvls %.0f GB/s", model_.alpha_us, model_.launch_us,
              model_.beta_gbps, model_.nvls_gbps);
    return HCCL_SUCCESS;
}

}  // namespace hcclb
