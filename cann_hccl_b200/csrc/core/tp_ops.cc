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

static std::map<Communicator *, std::map<std::string, TpWorkspace>> &workspaces()
{
    static std::map<Communicator *, std::map<std::string, TpWorkspace>> w;
    return w;
}

void Communicator::tp_release_workspaces()
{
    auto it = workspaces().find(this);
    if (it == workspaces().end()) return;
    for (auto &kv : it->second) alloc_->release(&kv.second.segs);
    workspaces().erase(it);
}

HcclResult Communicator::tp_workspace(const std::string &key, size_t data_bytes, int M, void **ws_out)
{
    auto &mine = workspaces()[this];
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
    // zero-copy source: when every rank's shard lies in registered symmetric memory at one common offset the peers pull it
    // from where it is; agreed once per (buffer, shape) so that all ranks take the same path
    std::vector<int> zh(nl, 0);
    std::vector<size_t> zo(nl, 0);
    bool zc = false;
    if (nranks_ > 1 && !user_segs_.empty()) {
        const size_t shard_bytes = (size_t)(M / nranks_) * K * 2;
        bool mine = true;
        for (int li = 0; li < nl && mine; ++li) {
            zh[li] = find_user_seg(li, x_shard[li], shard_bytes, &zo[li]);
            mine = zh[li] != 0 && (zo[li] & 15) == 0 && zh[li] == zh[0] && zo[li] == zo[0];
        }
        std::ostringstream zk;
        zk << "ag:" << x_shard[0] << ':' << M << ':' << K;
        auto zit = zc_agreed_.find(zk.str());
        if (zit == zc_agreed_.end()) {
            struct { uint32_t ok; int32_t h; uint64_t off; } me_v{mine ? 1u : 0u, zh[0], zo[0]};
            int agreed = mine ? 1 : 0;
            if (!all_local_) {
                std::vector<std::string> all;
                CHK_RET(exchange("zc/" + std::to_string(zc_agreed_.size()), std::string((const char *)&me_v, sizeof(me_v)), &all));
                for (auto &blob : all) {
                    decltype(me_v) o;
                    memcpy(&o, blob.data(), sizeof(o));
                    if (!o.ok || o.h != me_v.h || o.off != me_v.off) agreed = 0;
                }
            }
            zit = zc_agreed_.emplace(zk.str(), agreed).first;
        }
        zc = zit->second == 1;
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
    int ncomm = 8;  // the launcher drops them for a single rank
    if (const char *e = getenv("HCCL_TP_COMM_CTAS")) ncomm = std::max(1, atoi(e));
    return launch_tp_gemm(P.data(), A.data(), B.data(), nl, ncomm, stream);
}

HcclResult Communicator::tp_matmul_reduce_scatter(const void *const *h, const void *const *w, void *const *out, int M, int N, int K, void *stream)
{
    std::lock_guard<std::mutex> lk(op_mu_);
    CHK_RET(check_ready());
    CHK_RET_LOG(settings_.transport != TR_DEVICE, HCCL_E_NOT_SUPPORT, "fused tensor-parallel kernels need the device transport");
    int nl = nlocal();
    CHK_RET_LOG(nl > kTpMaxLocal, HCCL_E_NOT_SUPPORT, "at most %d virtual ranks per GPU for the fused kernels", kTpMaxLocal);
    CHK_RET_LOG(M % (128 * nranks_) != 0, HCCL_E_PARA, "M (%d) must be a multiple of 128 x ranks (%d)", M, 128 * nranks_);
    std::ostringstream key;
    key << "rs:" << M << ':' << N;
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
    return launch_tp_gemm(P.data(), A.data(), B.data(), nl, 0, stream);
}

}  // namespace hcclb
