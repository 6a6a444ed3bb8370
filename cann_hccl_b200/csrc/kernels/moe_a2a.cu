// MoE expert-parallel exchange for sm_100a: dispatch = every (token, expert) pair's activation row is stored straight
// into the expert owner's receive buffer over NVLink; combine = every token pulls its top-k expert output rows from the
// owners and forms the gate-weighted sum in fp32 while the rows arrive ("combine fused into the receive kernel").
// Counts are exchanged on the device (an all-gather of the per-expert histogram), so no host synchronisation sits on
// the path; the reference's AlltoAllV needs a host-side count exchange first (hccl_communicator.cc:3928
// RegressCalPreOp: all-gather + stream sync + D2H).
//
// Receive layout on the owner of local expert e: rows grouped [local expert][source rank][arrival order], so that the
// expert MLP sees one contiguous row range per expert (expert_offsets).
// Variants: MESH walks the pairs in token order, so all peers are written/read concurrently; PAIRWISE runs p-1 phases,
// phase i touching only rank (me + i) mod p (the traffic pattern of the reference's alltoallv_pairwise template).
// None of these kernels waits on another rank: ordering between ranks is provided by HcclBarrier launches around them.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "common/log.h"
#include "kernels/moe_a2a.h"

namespace hcclb {

namespace {

__global__ void moe_count_kernel(const int32_t *topk_idx, int64_t npairs, int n_experts, int32_t *hist, int32_t *pos)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < npairs; i += (int64_t)gridDim.x * blockDim.x) {
        int e = topk_idx[i];
        pos[i] = (e >= 0 && e < n_experts) ? atomicAdd(&hist[e], 1) : -1;
    }
}

// counts: [p][E] gathered histograms.  For this rank: base[e] = first receive row (on the owner of e) of my block for
// expert e; my own receive side: expert_offsets[El+1] and total rows.
__global__ void moe_offsets_kernel(const int32_t *counts, int p, int n_experts, int me, int32_t *base, int32_t *expert_offsets,
                                   int32_t *recv_rows, int64_t capacity_rows, int32_t *overflow)
{
    const int El = n_experts / p;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        int owner = e / El, e0 = owner * El;
        int64_t row = 0;
        for (int e2 = e0; e2 < e; ++e2)
            for (int i = 0; i < p; ++i) row += counts[i * n_experts + e2];
        for (int i = 0; i < me; ++i) row += counts[i * n_experts + e];
        base[e] = (int32_t)row;
    }
    if (threadIdx.x == 0) {
        int64_t row = 0;
        for (int el = 0; el < El; ++el) {
            expert_offsets[el] = (int32_t)row;
            for (int i = 0; i < p; ++i) row += counts[i * n_experts + me * El + el];
        }
        expert_offsets[El] = (int32_t)row;
        *recv_rows = (int32_t)row;
        if (row > capacity_rows) *overflow = 1;
    }
}

struct PeerTable {
    __nv_bfloat16 *ptr[kMaxRanks];
};

// one warp per (token, k) pair; rows are H bf16, H % 8 == 0
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const __nv_bfloat16 *x, const int32_t *topk_idx, const int32_t *pos,
                                                           const int32_t *base, int64_t npairs, int topk, int hidden, int n_experts, int p,
                                                           int me, int pairwise, PeerTable recv, int32_t *dst_row, int64_t capacity_rows)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int El = n_experts / p, nvec = hidden / 8;
    const int phases = pairwise ? p : 1;
    for (int ph = 0; ph < phases; ++ph) {
        const int only = pairwise ? (me + ph) % p : -1;
        for (int64_t i = warp; i < npairs; i += nwarps) {
            int e = topk_idx[i];
            if (e < 0 || e >= n_experts) continue;
            int owner = e / El;
            if (only >= 0 && owner != only) continue;
            int64_t row = (int64_t)base[e] + pos[i];
            if (lane == 0) dst_row[i] = (int32_t)row;
            if (row >= capacity_rows) continue;
            const uint4 *src = (const uint4 *)(x + (i / topk) * (int64_t)hidden);
            uint4 *dst = (uint4 *)(recv.ptr[owner] + row * (int64_t)hidden);
            for (int v = lane; v < nvec; v += 128) {  // four 16-byte vectors per lane in flight
                uint4 a = src[v], b, c, d;
                bool hb = v + 32 < nvec, hc = v + 64 < nvec, hd = v + 96 < nvec;
                if (hb) b = src[v + 32];
                if (hc) c = src[v + 64];
                if (hd) d = src[v + 96];
                dst[v] = a;
                if (hb) dst[v + 32] = b;
                if (hc) dst[v + 64] = c;
                if (hd) dst[v + 96] = d;
            }
        }
    }
}

// one warp per token: out[t] = sum_k gate[t,k] * y@owner(expert[t,k])[dst_row[t,k]]   (fp32 accumulate, fixed k order)
// The (owner pointer, gate) pairs of a token are resolved once; for every 16-byte column group the loads of up to eight
// k rows are issued together before the first one is consumed, so a lane keeps eight peer loads in flight.
constexpr int kCombineK = 8;
__global__ void __launch_bounds__(256) moe_combine_kernel(PeerTable y, const int32_t *topk_idx, const float *gates, const int32_t *dst_row,
                                                          int64_t tokens, int topk, int hidden, int n_experts, int p, int me, int pairwise,
                                                          __nv_bfloat16 *out, int64_t capacity_rows)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int El = n_experts / p, nvec = hidden / 8;
    for (int64_t t = warp; t < tokens; t += nwarps) {
        for (int k0 = 0; k0 < topk; k0 += kCombineK) {  // batches of eight k slots (one batch for top-8 routing)
            const uint4 *rowp[kCombineK];
            float g[kCombineK];
            int order[kCombineK];
            // pairwise order visits the slots by owner distance from this rank; mesh keeps the k order
            int n = 0;
            for (int ph = 0; ph < (pairwise ? p : 1); ++ph)
                for (int k = k0; k < topk && k < k0 + kCombineK; ++k) {
                    int e = topk_idx[t * topk + k];
                    if (e < 0 || e >= n_experts) continue;
                    int owner = e / El;
                    if (pairwise && owner != (me + ph) % p) continue;
                    int64_t row = dst_row[t * topk + k];
                    if (row < 0 || row >= capacity_rows) continue;
                    order[n] = k;
                    rowp[n] = (const uint4 *)(y.ptr[owner] + row * (int64_t)hidden);
                    g[n] = gates[t * topk + k];
                    ++n;
                }
            (void)order;
            for (int v = lane; v < nvec; v += 32) {
                uint4 r[kCombineK];
#pragma unroll
                for (int j = 0; j < kCombineK; ++j)
                    if (j < n) r[j] = rowp[j][v];
                float acc[8];
                if (k0 == 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
                } else {  // more than eight experts per token: continue from the partial sum written by the previous batch
                    uint4 o = ((const uint4 *)(out + t * (int64_t)hidden))[v];
                    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&o;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float2 f = __bfloat1622float2(h[i]);
                        acc[2 * i] = f.x;
                        acc[2 * i + 1] = f.y;
                    }
                }
#pragma unroll
                for (int j = 0; j < kCombineK; ++j) {
                    if (j < n) {
                        const __nv_bfloat162 *h = (const __nv_bfloat162 *)&r[j];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float2 f = __bfloat1622float2(h[i]);
                            acc[2 * i] += g[j] * f.x;
                            acc[2 * i + 1] += g[j] * f.y;
                        }
                    }
                }
                uint4 o;
                __nv_bfloat162 *h = (__nv_bfloat162 *)&o;
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                ((uint4 *)(out + t * (int64_t)hidden))[v] = o;
            }
        }
    }
}

HcclResult last_launch(const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        HLOG_ERROR("%s launch failed: %s", what, cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace

HcclResult moe_count(const int32_t *topk_idx, int64_t npairs, int n_experts, int32_t *hist, int32_t *pos, void *stream)
{
    cudaMemsetAsync(hist, 0, sizeof(int32_t) * n_experts, (cudaStream_t)stream);
    int blocks = (int)std::min<int64_t>((npairs + 255) / 256, 592);
    moe_count_kernel<<<std::max(1, blocks), 256, 0, (cudaStream_t)stream>>>(topk_idx, npairs, n_experts, hist, pos);
    return last_launch("moe_count");
}
HcclResult moe_offsets(const int32_t *counts, int p, int n_experts, int me, int32_t *base, int32_t *expert_offsets, int32_t *recv_rows,
                       int64_t capacity_rows, int32_t *overflow, void *stream)
{
    if (p < 1 || n_experts % p) return HCCL_E_PARA;
    moe_offsets_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(counts, p, n_experts, me, base, expert_offsets, recv_rows, capacity_rows, overflow);
    return last_launch("moe_offsets");
}
HcclResult moe_dispatch(const void *x, const int32_t *topk_idx, const int32_t *pos, const int32_t *base, int64_t tokens, int topk, int hidden,
                        int n_experts, int p, int me, int pairwise, void *const *recv_peers, int32_t *dst_row, int64_t capacity_rows, void *stream)
{
    if (hidden % 8 || p > kMaxRanks) return HCCL_E_PARA;
    PeerTable t;
    for (int q = 0; q < p; ++q) t.ptr[q] = (__nv_bfloat16 *)recv_peers[q];
    moe_dispatch_kernel<<<592, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x, topk_idx, pos, base, tokens * topk, topk, hidden, n_experts,
                                                              p, me, pairwise, t, dst_row, capacity_rows);
    return last_launch("moe_dispatch");
}
HcclResult moe_combine(void *const *y_peers, const int32_t *topk_idx, const float *gates, const int32_t *dst_row, int64_t tokens, int topk,
                       int hidden, int n_experts, int p, int me, int pairwise, void *out, int64_t capacity_rows, void *stream)
{
    if (hidden % 8 || p > kMaxRanks) return HCCL_E_PARA;
    PeerTable t;
    for (int q = 0; q < p; ++q) t.ptr[q] = (__nv_bfloat16 *)y_peers[q];
    moe_combine_kernel<<<592, 256, 0, (cudaStream_t)stream>>>(t, topk_idx, gates, dst_row, tokens, topk, hidden, n_experts, p, me, pairwise,
                                                             (__nv_bfloat16 *)out, capacity_rows);
    return last_launch("moe_combine");
}

}  // namespace hcclb
