// Host side of the fused tensor-parallel operators: symmetric workspaces (gathered X / partial-sum slots + flag words),
// per-workspace call epochs, and the launch of the fused sm_100a kernel (kernels/fused/tp_gemm_sm100.cu).
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include "common/log.h"
#include "core/communicator.h"
#include "kernels/fused/tp_gemm.h"

namespace hcclb {

struct TpWorkspace {
    std::vector<SymSegment> segs;  // per local rank
    size_t flag_bytes = 0, data_bytes = 0;
    uint64_t epoch = 0;
};

// Workspaces of all communicators of the process.  Communicators of different GPUs run on different threads
// (HcclCommInitAll): every access to the outer map holds ws_mu(); a communicator's own entries are only touched under its
// operation lock, so references into the inner map stay valid outside ws_mu().
static std::mutex &ws_mu()
{
    static std::mutex m;
    return m;
}
static std::map<Communicator *, std::map<std::string, TpWorkspace>> &workspaces()
{
    static std::map<Communicator *, std::map<std::string, TpWorkspace>> w;
    return w;
}

void Communicator::tp_release_workspaces()
{
    std::map<std::string, TpWorkspace> mine;
    {
        std::lock_guard<std::mutex> lk(ws_mu());
        auto it = workspaces().find(this);
        if (it == workspaces().end()) return;
        mine = std::move(it->second);
        workspaces().erase(it);
    }
    for (auto &kv : mine) alloc_->release(&kv.second.segs);
}

HcclResult Communicator::tp_workspace(const std::string &key, size_t data_bytes, int M, void **ws_out)
{
    std::map<std::string, TpWorkspace> *minep;
    {
        std::lock_guard<std::mutex> lk(ws_mu());
        minep = &workspaces()[this];  // std::map: the inner map's address survives insertions of other communicators
    }
    auto &mine = *minep;
    auto it = mine.find(key);
    if (it == mine.end()) {
        TpWorkspace w;
        w.flag_bytes = (tp_flag_words(M, nranks_) * 8 + 4095) / 4096 * 4096;
        w.data_bytes = data_bytes;
        StateGuard guard(state_, CS_BUILDING);
        CHK_RET(alloc_->alloc(w.flag_bytes + data_bytes, false, &w.segs));
        it = mine.emplace(key, std::move(w)).first;
    }
    *ws_out = &it->second;
    return HCCL_SUCCESS;
}

static void fill_common(TpGemmParams &P, int mode, int M, int N, int K, int rank, int nranks, uint64_t epoch, uint64_t timeout_ns,
                        DevStatus *status, uint32_t *fail_word)
{
    memset(&P, 0, sizeof(P));
    P.mode = mode; P.M = M; P.N = N; P.K = K; P.rank = rank; P.nranks = nranks; P.epoch = epoch; P.timeout_ns = timeout_ns;
    P.status = status; P.fail_word = fail_word;
}

HcclResult gemm_bf16_plain(const void *A, const void *B, void *C, int M, int N, int K, void *stream)
{
    TpGemmParams P;
    fill_common(P, TP_MODE_PLAIN, M, N, K, 0, 1, 1, 10000000000ull, nullptr, nullptr);
    P.C = (__nv_bfloat16 *)C;
    P.ldc = N;
    const void *a[1] = {A}, *b[1] = {B};
    return launch_tp_gemm(&P, a, b, 1, 0, stream);
}

HcclResult Communicator::tp_all_gather_matmul(const void *const *x_shard, const void *const *w, void *const *y, int M, int N, int K, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    CHK_RET_LOG(settings_.transport != TR_DEVICE, HCCL_E_NOT_SUPPORT, "fused tensor-parallel kernels need the device transport");
    int nl = nlocal();
    CHK_RET_LOG(nl > kTpMaxLocal, HCCL_E_NOT_SUPPORT, "at most %d virtual ranks per GPU for the fused kernels", kTpMaxLocal);
    CHK_RET_LOG(M % (128 * nranks_) != 0, HCCL_E_PARA, "M (%d) must be a multiple of 128 x ranks (%d)", M, 128 * nranks_);
    std::ostringstream key;
    key << "ag:" << M << ':' << K;
    void *wsp = nullptr;
    CHK_RET(tp_workspace(key.str(), (size_t)M * K * 2, M, &wsp));
    TpWorkspace &ws = *(TpWorkspace *)wsp;
    ++ws.epoch;
    // zero-copy source: a shard that lies in registered symmetric memory is pulled by the peers from where it is.  Decided
    // from this rank's own lookup: symmetric memory is used with the same (allocation, offset) on every rank by contract,
    // so no per-call agreement round (in which a rank could wait alone) is needed.
    std::vector<int> zh(nl, 0);
    std::vector<size_t> zo(nl, 0);
    bool zc = false;
    if (nranks_ > 1 && !user_segs_.empty()) {
        const size_t shard_bytes = (size_t)(M / nranks_) * K * 2;
        zc = true;
        for (int li = 0; li < nl && zc; ++li) {
            zh[li] = find_user_seg(li, x_shard[li], shard_bytes, &zo[li]);
            zc = zh[li] != 0 && (zo[li] & 15) == 0 && zh[li] == zh[0] && zo[li] == zo[0];
        }
    }
    StateGuard guard(state_, CS_INUSE);
    std::vector<TpGemmParams> P(nl);
    std::vector<const void *> A(nl), B(nl);
    for (int li = 0; li < nl; ++li) {
        fill_common(P[li], TP_MODE_AG, M, N, K, ctx_[li].rank, nranks_, ws.epoch, ctx_[li].timeout_ns, status_[li], ctx_[li].exit_counter + 1);
        P[li].C = (__nv_bfloat16 *)y[li];
        P[li].ldc = N;
        P[li].x_shard = (const __nv_bfloat16 *)x_shard[li];
        for (int q = 0; q < nranks_; ++q) {
            P[li].flags[q] = (uint64_t *)ws.segs[li].peer[q];
            P[li].xfull[q] = (__nv_bfloat16 *)(ws.segs[li].peer[q] + ws.flag_bytes);
            if (zc) P[li].x_peer[q] = (const __nv_bfloat16 *)(user_segs_[zh[li]][li].peer[q] + zo[li]);
        }
        A[li] = P[li].xfull[ctx_[li].rank];
        B[li] = w[li];
    }
    stats_.launches++;
    stats_.ops[COLL_ALLGATHER]++;
    // data-movement CTAs (the launcher drops them for a single rank).  Read once per process: the completion counters of a
    // workspace count these CTAs over all calls, so the number must not change between two calls on the same shape.
    static const int ncomm_env = [] { const char *e = getenv("HCCL_TP_COMM_CTAS"); return e ? std::max(1, atoi(e)) : 8; }();
    int ncomm = ncomm_env;
    HcclResult rc = launch_tp_gemm(P.data(), A.data(), B.data(), nl, ncomm, stream);
    if (rc != HCCL_SUCCESS) --ws.epoch;  // rejected before any kernel ran: the counters still stand at the previous call
    return rc;
}

HcclResult Communicator::tp_matmul_reduce_scatter(const void *const *h, const void *const *w, void *const *out, int M, int N, int K, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    CHK_RET_LOG(settings_.transport != TR_DEVICE, HCCL_E_NOT_SUPPORT, "fused tensor-parallel kernels need the device transport");
    int nl = nlocal();
    CHK_RET_LOG(nl > kTpMaxLocal, HCCL_E_NOT_SUPPORT, "at most %d virtual ranks per GPU for the fused kernels", kTpMaxLocal);
    CHK_RET_LOG(M % (128 * nranks_) != 0, HCCL_E_PARA, "M (%d) must be a multiple of 128 x ranks (%d)", M, 128 * nranks_);
    if (nranks_ == 1) {
        // nothing to reduce or scatter: the product goes straight to the output, without a pass through a receive slot
        stats_.launches++;
        stats_.ops[COLL_REDUCE_SCATTER]++;
        return gemm_bf16_plain(h[0], w[0], out[0], M, N, K, stream);
    }
    std::ostringstream key;
    key << "rs:" << M << ':' << N << ':' << K;  // the panel layout of the completion counters depends on K as well
    void *wsp = nullptr;
    CHK_RET(tp_workspace(key.str(), (size_t)M * N * 2, M, &wsp));
    TpWorkspace &ws = *(TpWorkspace *)wsp;
    ++ws.epoch;
    StateGuard guard(state_, CS_INUSE);
    std::vector<TpGemmParams> P(nl);
    std::vector<const void *> A(nl), B(nl);
    for (int li = 0; li < nl; ++li) {
        fill_common(P[li], TP_MODE_RS, M, N, K, ctx_[li].rank, nranks_, ws.epoch, ctx_[li].timeout_ns, status_[li], ctx_[li].exit_counter + 1);
        P[li].out = (__nv_bfloat16 *)out[li];
        for (int q = 0; q < nranks_; ++q) {
            P[li].flags[q] = (uint64_t *)ws.segs[li].peer[q];
            P[li].partial[q] = (__nv_bfloat16 *)(ws.segs[li].peer[q] + ws.flag_bytes);
        }
        A[li] = h[li];
        B[li] = w[li];
    }
    stats_.launches++;
    stats_.ops[COLL_REDUCE_SCATTER]++;
    HcclResult rc = launch_tp_gemm(P.data(), A.data(), B.data(), nl, 0, stream);
    if (rc != HCCL_SUCCESS) --ws.epoch;  // rejected before any kernel ran: the counters still stand at the previous call
    return rc;
}

}  // namespace hcclb
