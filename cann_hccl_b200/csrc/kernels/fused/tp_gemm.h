// Launch interface of the fused tensor-parallel GEMM kernels (kernels/fused/tp_gemm_sm100.cu).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include "algo/plan.h"
namespace hcclb {
enum TpMode : int { TP_MODE_PLAIN = 0, TP_MODE_AG = 1, TP_MODE_RS = 2 };
constexpr int kTpMaxLocal = 4;   // virtual ranks of one GPU that one cooperative launch can run (single-GPU validation)
struct alignas(64) TpGemmParams {
    CUtensorMap tmA, tmB;             // A [M,K] and B [N,K], both K-major bf16, this GPU's own memory
    CUtensorMap tmX;                  // AG: this rank's own shard [M/p, K] in the caller's buffer
    __nv_bfloat16 *C;                 // PLAIN / AG: output [M, ldc]
    int ldc;
    int M, N, K;
    int mode, rank, nranks;
    int n_gemm_ctas;                  // CTAs [0, n_gemm_ctas) compute; the rest move data
    uint64_t epoch;                   // call count on this workspace, from 1
    uint64_t timeout_ns;
    const __nv_bfloat16 *x_shard;     // AG: this rank's rows [M/p, K]
    const __nv_bfloat16 *x_peer[kMaxRanks]; // AG, optional: rank q's x_shard as mapped here (registered symmetric memory): peers pull from it, nothing is staged
    __nv_bfloat16 *xfull[kMaxRanks];  // AG: gathered X [M,K] of rank q (symmetric); A's tensor map covers xfull[rank]
    __nv_bfloat16 *partial[kMaxRanks];// RS: receive area of rank q: p slots of [M/p, N]
    __nv_bfloat16 *out;               // RS: this rank's reduced rows [M/p, N]
    uint64_t *flags[kMaxRanks];       // flag words of rank q (symmetric)
    DevStatus *status;                // host-mapped status block (may be null)
    uint32_t *fail_word;              // device word: first failure of this rank
};
struct TpGemmParamsArray {
    TpGemmParams r[kTpMaxLocal];
};
// Flag words a rank needs for AG ( 2 x [p], chunk_ready[M/128], ready[p x 32 data-movement CTAs] ) and RS ( count[M/128 row
// blocks x panels], done[p] ); up to 64 panels.
inline size_t tp_flag_words(int M, int nranks) { return (size_t)4 * nranks + (size_t)(M / 128) * 64 + 64 + (size_t)nranks * 32; }
// Fills the tensor maps and launches.  `A` / `B` per local rank.  n_comm_ctas data-movement CTAs per rank.
HcclResult launch_tp_gemm(TpGemmParams *P, const void *const *A, const void *const *B, int nlocal, int n_comm_ctas, void *stream);
size_t tp_gemm_smem_bytes();
void tp_gemm_launch_counts(uint64_t *single, uint64_t *pair);
}  // namespace hcclb
