// MoE dispatch / combine kernels (kernels/moe_a2a.cu).  All pointers are device pointers; peer tables are host arrays
// of p device pointers (rank q's buffer as mapped on this rank).
#pragma once
#include <algorithm>
#include "common/base.h"
namespace hcclb {
HcclResult moe_count(const int32_t *topk_idx, int64_t npairs, int n_experts, int32_t *hist, int32_t *pos, void *stream);
HcclResult moe_offsets(const int32_t *counts, int p, int n_experts, int me, int32_t *base, int32_t *expert_offsets, int32_t *recv_rows,
                       int64_t capacity_rows, int32_t *overflow, void *stream);
HcclResult moe_dispatch(const void *x, const int32_t *topk_idx, const int32_t *pos, const int32_t *base, int64_t tokens, int topk, int hidden,
                        int n_experts, int p, int me, int pairwise, void *const *recv_peers, int32_t *dst_row, int64_t capacity_rows, void *stream);
HcclResult moe_combine(void *const *y_peers, const int32_t *topk_idx, const float *gates, const int32_t *dst_row, int64_t tokens, int topk,
                       int hidden, int n_experts, int p, int me, int pairwise, void *out, int64_t capacity_rows, void *stream);
}  // namespace hcclb
