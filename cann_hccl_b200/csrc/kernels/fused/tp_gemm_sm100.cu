// Fused tensor-parallel GEMM kernels for sm_100a (bf16 in, fp32 accumulate in TMEM, bf16 out).
//
//   mode PLAIN : C[M,N] = A[M,K] * B[N,K]^T                                   (building block, TP = 1)
//   mode AG    : all-gather(X shards) -> Y = X * W^T   (column-parallel layer; X sharded by rows over the ranks)
//   mode RS    : P = H * W^T -> reduce-scatter(P) by rows  (row-parallel layer; every rank ends with its row block)
//
// One persistent kernel does the transfer and the math, one CTA per SM:
//   warp 0    feeds a 4-stage shared-memory ring with TMA (cp.async.bulk.tensor, 128-byte swizzle, never multicast,
//             always from this GPU's own memory);
//   warp 1    issues tcgen05.mma (128x256x16, cta_group::1) into one of two 256-column TMEM accumulators;
//             pair variant (tp_gemm_pair_kernel, clusters of two CTAs, used when every rank's rows are a multiple of
//             256): the two CTAs of a cluster own the upper and lower 128 rows of a 256x256 tile, each loads its own
//             rows of A and HALF of the tile's B rows (plain, non-multicast TMA loads that complete on the leader
//             CTA's barrier), and the leader's warp 1 issues tcgen05.mma.cta_group::2 (256x256x16) which reads both
//             CTAs' shared memory and writes both CTAs' TMEM: B crosses L2 -> SM once per pair instead of once per CTA
//             and a stage shrinks from 48 to 32 KB (six stages instead of four);
//   warps 2-5 drain the other accumulator with tcgen05.ld, convert to bf16 and send each 128-byte row piece off with a
//             bulk asynchronous store (to local memory, or in RS mode straight into the owner rank's receive slot
//             over NVLink, followed by a counter increment there);
//   AG        a handful of extra CTAs move data instead: they stage this rank's shard into its slot of the symmetric
//             X buffer and pull the peers' shards over NVLink with bulk asynchronous copies (peer global -> shared ->
//             local global, six 32 KB pieces in flight per CTA) in the order in which the GEMM consumes the 128-row
//             blocks; the TMA producer waits on a per-block flag.
//   RS tail   after its last tile every CTA sums receive slots (fp32, fixed rank order) for the (row block, n tile)
//             items whose partial tiles have arrived from all ranks.
// Tiles are rasterised in L2-sized panels of n tiles so that a panel's weights are read from HBM once.
// Role of the reference's MC2 hooks (framework/op_base/src/op_base.cc:3137-3284: resources exported so that a fused
// matmul+communication kernel can be written elsewhere); here the fused kernels are part of the library.
//
// Every wait (mbarrier, flag, counter) is bounded: after the limit the waiting thread raises a CTA-wide failure word,
// every role leaves its loop, outstanding bulk copies are drained, TMEM is freed and the kernel returns with an
// error code in the status block.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <atomic>
#include <mutex>
#include <algorithm>
#include <cstring>
#include "common/env.h"
#include "common/log.h"
#include "core/device_api.h"
#include "kernels/fused/tp_gemm.h"
#include "kernels/fused/tp_gemm_noalloc.h"
#include "kernels/prims.cuh"

namespace hcclb {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kStagesPair = 6;                        // pair variant: a stage holds 128 rows of A and 128 rows of B
constexpr int kMaxStages = kStagesPair;
constexpr int kMaxPanels = 60;
constexpr int kMaxCommCtas = 32;  // data-movement CTAs per rank (AG), bound of the per-CTA ready words
constexpr int kThreads = 256;  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warps 6-7 move data between GPUs (AG)
constexpr uint32_t kABytes = BM * BK * 2, kBBytes = BN * BK * 2, kStageBytes = kABytes + kBBytes;
constexpr uint32_t kBBytesPair = kBBytes / 2, kStageBytesPair = kABytes + kBBytesPair;
static_assert(kStagesPair * kStageBytesPair <= kStages * kStageBytes, "both variants share the tile buffers");
constexpr uint32_t kTmemCols = 512;
constexpr int kCommBuf = 32 * 1024, kCommDepth = 6;  // bulk-copy ring of a data-movement CTA (lives in the tile buffers)
constexpr int kEpiCols = 64, kEpiStride = kEpiCols * 2 + 16;  // epilogue chunk: 64 bf16 per row, padded against bank conflicts
constexpr uint64_t kPairWaitNs = 4000000000ull;     // pair variant: longest wait on a barrier that the other CTA completes
constexpr uint32_t kSpinLimit = 1u << 28;            // iterations of an mbarrier poll before it gives up (seconds)

struct SharedStorage {
    alignas(1024) uint8_t tiles[kStages * kStageBytes];
    alignas(16) uint8_t epi[128 * kEpiStride];          // one 128-byte (+16 pad) row slot per epilogue thread
    alignas(8) uint64_t full_bar[kMaxStages];
    uint64_t empty_bar[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t comm_bar[kCommDepth];
    uint32_t tmem_base;
    uint32_t fail;
    uint32_t gemm_done;      // RS: the epilogue has published this CTA's last tile
    uint32_t early_go[2];    // RS: decision of the early reducer's leader for its next item (by item parity)
    uint32_t early_count;    // RS: items this CTA's early reducer finished before the GEMM ended
};

// ---------------------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another role already failed.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *fail)
{
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 1023) == 1023 && *fail) return false;
    }
    *fail = HCCL_E_TIMEOUT;
    return false;
}
// Cluster-scope forms for the pair variant: barriers that the other CTA of the pair (its threads, its TMA loads or the
// leader's multicast commits) completes.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
template <bool kCluster>
__device__ __forceinline__ bool mbar_wait_t(uint64_t *bar, uint32_t parity, volatile uint32_t *fail)
{
    if constexpr (!kCluster) {
        return mbar_wait(bar, parity, fail);
    } else {
        // the other CTA of the pair learns of a failure only through its own waits: bound them by time, a few seconds
        uint64_t t0 = 0;
        for (uint32_t it = 0; it < kSpinLimit; ++it) {
            if (mbar_try_wait_cluster(bar, parity)) return true;
            if ((it & 1023) == 1023) {
                if (*fail) return false;
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > kPairWaitNs) break;
            }
        }
        *fail = HCCL_E_TIMEOUT;
        return false;
    }
}
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_u32(uint32_t cta_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load of the pair variant: the data lands in this CTA's shared memory, the bytes are counted on the barrier at
// `bar_cluster_addr`, which may belong to the other CTA of the pair (no multicast: one load, one destination).
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, uint32_t bar_cluster_addr, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *dst, const void *src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
    return pred != 0;
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(const void *ptr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(ptr) & 0x3FFFF) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                            // leading-dimension byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride-dimension byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, N = 256, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate)
{
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Pair variant: D fp32, A and B bf16 K-major, N = 256, M = 256 (128 rows per CTA); issued by one thread of the leader CTA.
constexpr uint32_t kInstrDescPair = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate)
{
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDescPair), "r"(accumulate), "r"(0u) : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far are complete.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar)
{
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
        "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(uint32_t a, uint32_t b)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(a), __uint_as_float(b));
    return *(uint32_t *)&v;
}
__device__ __forceinline__ void red_add_release_sys(uint64_t *p, uint64_t v)
{
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu(uint64_t *p, uint64_t v)
{
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(uint64_t *p, uint64_t v)
{
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_gpu(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait on a global word (device or system scope); returns false after the time limit or a CTA failure.
__device__ __forceinline__ bool wait_word_ge(const uint64_t *p, uint64_t want, bool sys, uint64_t deadline, volatile uint32_t *fail)
{
    for (uint32_t it = 0;; ++it) {
        uint64_t v = sys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
        if (v >= want) return true;
        if ((it & 63) == 63) {
            if (*fail) return false;
            if (global_timer_ns() > deadline) { *fail = HCCL_E_TIMEOUT; return false; }
        }
    }
}

__device__ __forceinline__ void report(const TpGemmParams &P, uint32_t code, int where)
{
    if (!P.fail_word) return;
    if (atomicCAS(P.fail_word, 0u, code) != 0u) return;
    if (!P.status) return;  // no host-mapped status block (allocation-free entry): the failure word is the record
    DevStatus *s = P.status;
    s->step = (uint32_t)where;
    s->peer = -1;
    s->chan = blockIdx.x;
    s->seq = P.epoch;
    __threadfence_system();
    *(volatile uint32_t *)&s->code = code;
}

// Logical tile index -> (m tile, n tile, panel).  The n tiles are cut into panels narrow enough for the panel's
// weights (panel width x 256 rows x K) to stay in L2 while the m tiles of a shard stream past; inside a panel tiles
// walk n fastest.
__device__ __forceinline__ int panel_width(const TpGemmParams &P, int n_tiles)
{
    long long w = (40ll << 20) / ((long long)BN * P.K * 2);
    if (P.mode == TP_MODE_RS) {
        // A panel's receive slots are summed while the next panel is computed, so only the last panel is left for the tail:
        // narrower panels shorten that tail.  Every panel streams A once more, hence no more than about N / 1024 of them.
        int target = P.N / 1024;
        target = target < 1 ? 1 : (target > 8 ? 8 : target);
        const long long wr = (n_tiles + target - 1) / target;
        if (wr < w) w = wr;
    }
    const long long wmin = (n_tiles + kMaxPanels - 1) / kMaxPanels;  // the flag area holds kMaxPanels counters per row block
    if (w < wmin) w = wmin;
    if (w < 1) w = 1;
    if (w > n_tiles) w = n_tiles;
    return (int)w;
}
__device__ __forceinline__ void tile_coords(const TpGemmParams &P, int t, int n_tiles, int m_tiles, int pw, int &mt, int &nt, int &panel)
{
    // rows are handled shard by shard (one rank's row blocks at a time, all panels), so that the transfer of the next
    // shard has the whole compute time of the current one; without communication there is a single "shard"
    // RS pushes asynchronously and keeps the L2-friendliest order.  AG always goes shard by shard: walking the global
    // panel order instead asks for every remote shard within the first panel, i.e. for more NVLink bandwidth than the
    // data-movement CTAs deliver (measured on 8 GPUs: 0.65 ms against 0.50 ms for 8192 x 3584 x 8192).
    const bool comm = P.mode == TP_MODE_AG && P.nranks > 1;
    const int per = comm ? m_tiles / P.nranks : m_tiles;  // m tiles per shard
    const int tiles_per_shard = per * n_tiles;
    const int sidx = t / tiles_per_shard, r1 = t - sidx * tiles_per_shard;
    const int per_panel = per * pw;
    panel = r1 / per_panel;
    const int n0 = panel * pw;
    const int w = n_tiles - n0 < pw ? n_tiles - n0 : pw;  // the last panel may be narrower
    const int r2 = r1 - panel * per_panel;
    const int ml = r2 / w;
    nt = n0 + r2 % w;
    if (P.mode == TP_MODE_PLAIN || P.nranks == 1) { mt = ml; return; }
    if (P.mode == TP_MODE_RS) {  // the next rank's rows first so that remote partial tiles leave early; my own rows last
        mt = (ml + ((P.rank + 1) % P.nranks) * (m_tiles / P.nranks)) % m_tiles;
        return;
    }
    // AG: own shard first (read straight from the caller's buffer), then the ranks after me in fetch order
    mt = ((sidx + P.rank) % P.nranks) * per + ml;
}

// ---------------------------------------------------------------------------------------------- comm CTAs
// Copy `bytes` from src (any global memory, possibly a peer's) to dst (local global) with bulk asynchronous copies
// through the shared-memory ring: loads run kCommDepth-1 pieces ahead of the stores.  One thread drives it.
// `g` counts pieces over the kernel's lifetime (ring slot = g % depth, mbarrier parity = (g / depth) & 1).
// On return every piece has been loaded and its store issued; the caller waits for the stores (wait_group 0).
__device__ bool bulk_copy(SharedStorage &S, uint8_t *dst, const uint8_t *src, uint64_t bytes, uint32_t &g, volatile uint32_t *fail)
{
    const uint32_t np = (uint32_t)((bytes + kCommBuf - 1) / kCommBuf), g0 = g;
    auto piece_len = [&](uint32_t i) { return (uint32_t)(((uint64_t)(i + 1) * kCommBuf <= bytes) ? kCommBuf : (bytes - (uint64_t)i * kCommBuf)); };
    auto issue_load = [&](uint32_t i) {
        uint32_t slot = (g0 + i) % kCommDepth, len = piece_len(i);
        mbar_expect_tx(&S.comm_bar[slot], len);
        bulk_g2s(S.tiles + (size_t)slot * kCommBuf, src + (uint64_t)i * kCommBuf, len, &S.comm_bar[slot]);
    };
    for (uint32_t i = 0; i < np && i < (uint32_t)(kCommDepth - 1); ++i) issue_load(i);
    for (uint32_t i = 0; i < np; ++i) {
        uint32_t slot = (g0 + i) % kCommDepth, parity = ((g0 + i) / kCommDepth) & 1;
        if (!mbar_wait(&S.comm_bar[slot], parity, fail)) return false;
        bulk_s2g(dst + (uint64_t)i * kCommBuf, S.tiles + (size_t)slot * kCommBuf, piece_len(i));
        bulk_commit();
        bulk_wait_read<1>();  // the store of piece i-1 has read its slot: that slot takes the next load
        uint32_t n = i + kCommDepth - 1;
        if (n < np) issue_load(n);
    }
    g = g0 + np;
    return true;
}

// Flag words of a rank in AG mode (uint64):
//   [src]          (unused)
//   [p + src]      done : comm CTAs of src that finished pulling from this rank (epoch * nc when complete)
//   [2p + m tile]  local: epoch once the rows of that m tile are in this rank's gathered X
//   [2p + m_tiles + src * kMaxCommCtas + c]  ready: m tiles of src's shard that src's comm CTA c has made available, counted
//                  over all calls.  Comm CTA c of every rank handles the tiles c, c + nc, ... of each shard, so the puller of
//                  a tile and its provider talk through one word and a pull starts as soon as that one tile is there.
__device__ void comm_role_ag(const TpGemmParams &P, SharedStorage &S, int c, int nc)
{
    const int p = P.nranks, me = P.rank;
    const int m_tiles = P.M / BM, per = m_tiles / p;
    const uint64_t tile_bytes = (uint64_t)P.K * 2 * BM;
    uint64_t *myflags = P.flags[me];
    const uint64_t deadline = global_timer_ns() + P.timeout_ns;
    volatile uint32_t *fail = &S.fail;
    if (threadIdx.x != 0) return;  // one thread drives the bulk copies
    if (p == 1) return;            // nobody to serve and nothing to fetch: the GEMM reads the caller's rows directly
    uint32_t g = 0;
    const uint64_t mine_per_call = c < per ? (uint64_t)(per - c + nc - 1) / nc : 0;  // tiles of a shard that comm CTA c handles
    const uint64_t ready_base = 2 * (uint64_t)p + m_tiles + c;
    // zero-copy source: every rank's shard sits in registered symmetric memory, so the peers read it where it is
    const bool zc = P.x_peer[(me + 1) % p] != nullptr;
    if (zc) {
        // stream order made my shard valid before this kernel began: tell the peers at once
        if (mine_per_call)
            for (int q = 0; q < p; ++q)
                if (q != me) red_add_release_sys(P.flags[q] + ready_base + (uint64_t)me * kMaxCommCtas, mine_per_call);
    } else {
        // the peers' pulls of the previous call from my slot must be over before I overwrite it
        for (int q = 0; q < p; ++q)
            if (q != me && !wait_word_ge(myflags + p + q, (P.epoch - 1) * (uint64_t)nc, true, deadline, fail)) { report(P, *fail, 100 + q); return; }
        // stage my shard into my slot of the gathered buffer: m tiles [me*per, (me+1)*per), split over the comm CTAs
        for (int j = c; j < per; j += nc) {
            int mt = me * per + j;
            if (!bulk_copy(S, (uint8_t *)P.xfull[me] + (uint64_t)mt * tile_bytes, (const uint8_t *)P.x_shard + (uint64_t)j * tile_bytes, tile_bytes, g, fail)) { report(P, *fail, 200); return; }
            bulk_wait_all<0>();
            fence_proxy_async();
            for (int q = 0; q < p; ++q)
                if (q != me) red_add_release_sys(P.flags[q] + ready_base + (uint64_t)me * kMaxCommCtas, 1);  // the peers may pull it
        }
    }
    // pull the peers' shards in the order in which the GEMM consumes them
    for (int i = 1; i < p; ++i) {
        int q = (me + i) % p;
        uint64_t k = 0;
        for (int j = c; j < per; j += nc, ++k) {
            int mt = q * per + j;
            if (!wait_word_ge(myflags + ready_base + (uint64_t)q * kMaxCommCtas, (P.epoch - 1) * mine_per_call + k + 1, true, deadline, fail)) { report(P, *fail, 300 + q); return; }
            const uint8_t *src = zc ? (const uint8_t *)P.x_peer[q] + (uint64_t)j * tile_bytes : (const uint8_t *)P.xfull[q] + (uint64_t)mt * tile_bytes;
            if (!bulk_copy(S, (uint8_t *)P.xfull[me] + (uint64_t)mt * tile_bytes, src, tile_bytes, g, fail)) { report(P, *fail, 400 + q); return; }
            bulk_wait_all<0>();
            fence_proxy_async();
            st_release_gpu(myflags + 2 * p + mt, P.epoch);
        }
    }
    // this CTA no longer reads any peer's memory
    for (int q = 0; q < p; ++q)
        if (q != me) red_add_release_sys(P.flags[q] + p + me, 1);
    // zero-copy: the caller may overwrite its shard once this kernel is over, so the peers' pulls have to be over by then
    if (zc && c == 0)
        for (int q = 0; q < p; ++q)
            if (q != me && !wait_word_ge(myflags + p + q, P.epoch * (uint64_t)nc, true, deadline, fail)) { report(P, *fail, 700 + q); return; }
}

__device__ __forceinline__ uint64_t rs_done_index(const TpGemmParams &P, int per, int npanels) { return (uint64_t)P.nranks * per * npanels; }

// Flag words of a rank in RS mode (uint64):
//   [(src * per + j) * panels + panel]  n tiles of panel `panel` of this rank's row block j delivered by src
//   [p * per * panels + o]  CTAs of owner o that finished reducing (epoch * G when complete): o's slots may be rewritten
// Reduce item = (panel, my row block j, n tile) -> 128 x 256 outputs, summed over the p receive slots in fp32 in rank
// order once all sources have delivered that panel of block j.  Items are ordered like the GEMM's production (panel major,
// then row block, then n tile) and dealt round-robin to the CTAs.  While the GEMM runs, the CTA's two spare warps reduce
// the items whose inputs are complete (everything but the last panel, as a rule); after its GEMM tiles the whole CTA
// finishes the rest.
struct RsItem { int panel, j, nt, w; };
__device__ __forceinline__ RsItem rs_item(int item, int per, int n_tiles, int pw)
{
    RsItem it;
    int rem = item;
    it.panel = 0;
    for (;; ++it.panel) {
        int n0p = it.panel * pw, wp = (n_tiles - n0p < pw) ? n_tiles - n0p : pw;
        if (rem < per * wp) break;
        rem -= per * wp;
    }
    const int n0 = it.panel * pw;
    it.w = (n_tiles - n0 < pw) ? n_tiles - n0 : pw;
    it.j = rem / it.w;
    it.nt = n0 + rem % it.w;
    return it;
}

// Sums one item with `nthr` threads (lid = this thread's index among them).  Every thread sums four 16-byte vectors at a
// time, two slots per round: eight loads are in flight before the first add whatever the rank count (one load at a time
// would leave the reduction latency-bound).
__device__ __forceinline__ void rs_reduce_item(const TpGemmParams &P, const RsItem &it, int lid, int nthr)
{
    const int p = P.nranks, me = P.rank;
    const uint64_t slot_elems = (uint64_t)(P.M / p) * P.N;  // one source's partial rows for me
    constexpr int vec_per_row = BN / 8, kVec = 4;
    for (int v0 = lid; v0 < BM * vec_per_row; v0 += kVec * nthr) {
        uint64_t eoff[kVec];
        float acc[kVec][8];
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
            const int v = v0 + i * nthr;  // BM * vec_per_row is a multiple of kVec * nthr
            eoff[i] = ((uint64_t)it.j * BM + v / vec_per_row) * P.N + (uint64_t)it.nt * BN + (uint64_t)(v % vec_per_row) * 8;
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[i][k] = 0.f;
        }
        for (int q0 = 0; q0 < p; q0 += 2) {
            uint4 x[kVec][2];
            const bool two = q0 + 1 < p;
#pragma unroll
            for (int i = 0; i < kVec; ++i) {
                x[i][0] = ld_stream((const uint4 *)(P.partial[me] + (uint64_t)q0 * slot_elems + eoff[i]));
                x[i][1] = two ? ld_stream((const uint4 *)(P.partial[me] + (uint64_t)(q0 + 1) * slot_elems + eoff[i])) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int i = 0; i < kVec; ++i)
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&x[i][u];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float2 f = __bfloat1622float2(h[k]);
                        acc[i][2 * k] += f.x;
                        acc[i][2 * k + 1] += f.y;
                    }
                }
        }
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
            uint4 o;
            o.x = pack_bf16(__float_as_uint(acc[i][0]), __float_as_uint(acc[i][1]));
            o.y = pack_bf16(__float_as_uint(acc[i][2]), __float_as_uint(acc[i][3]));
            o.z = pack_bf16(__float_as_uint(acc[i][4]), __float_as_uint(acc[i][5]));
            o.w = pack_bf16(__float_as_uint(acc[i][6]), __float_as_uint(acc[i][7]));
            *(uint4 *)(P.out + eoff[i]) = o;
        }
    }
}

// The two spare warps (64 threads) while the GEMM runs.  Their leader polls the p delivery counters of the next item; it
// gives up as soon as the CTA's GEMM is over (the whole CTA is faster from there) or a failure is flagged.
__device__ void reduce_early_rs(const TpGemmParams &P, SharedStorage &S, int pw, int npanels)
{
    const int p = P.nranks, me = P.rank;
    const int m_tiles = P.M / BM, per = m_tiles / p, n_tiles = P.N / BN;
    const uint64_t *myflags = P.flags[me];
    const int lid = threadIdx.x - (kThreads - 64);
    const int items = per * n_tiles;
    uint32_t done = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++done) {
        const RsItem it = rs_item(item, per, n_tiles, pw);
        if (lid == 0) {
            uint32_t go = 0;
            for (;;) {
                if (*(volatile uint32_t *)&S.gemm_done || *(volatile uint32_t *)&S.fail) break;
                int q = 0;
                for (; q < p; ++q)
                    if (ld_acquire_sys(myflags + ((uint64_t)q * per + it.j) * npanels + it.panel) < P.epoch * (uint64_t)it.w) break;
                if (q == p) { go = 1; break; }
                __nanosleep(200);
            }
            *(volatile uint32_t *)&S.early_go[done & 1] = go;
        }
        asm volatile("bar.sync 2, 64;" ::: "memory");
        if (!*(volatile uint32_t *)&S.early_go[done & 1]) break;
        rs_reduce_item(P, it, lid, 64);
    }
    if (lid == 0) S.early_count = done;
}

__device__ void reduce_tail_rs(const TpGemmParams &P, SharedStorage &S, int pw, int npanels)
{
    const int p = P.nranks, me = P.rank;
    const int m_tiles = P.M / BM, per = m_tiles / p, n_tiles = P.N / BN;
    uint64_t *myflags = P.flags[me];
    const uint64_t deadline = global_timer_ns() + P.timeout_ns;
    volatile uint32_t *fail = &S.fail;
    const int items = per * n_tiles;
    for (int item = blockIdx.x + (int)S.early_count * gridDim.x; item < items; item += gridDim.x) {
        const RsItem it = rs_item(item, per, n_tiles, pw);
        if (threadIdx.x < p) {
            if (!wait_word_ge(myflags + ((uint64_t)threadIdx.x * per + it.j) * npanels + it.panel, P.epoch * (uint64_t)it.w, true, deadline, fail)) report(P, *fail, 500 + threadIdx.x);
        }
        if (__syncthreads_or((int)*fail)) return;
        rs_reduce_item(P, it, threadIdx.x, blockDim.x);
        __syncthreads();
    }
    // this CTA is done reading my receive slots: sources may overwrite them in the next call once every CTA said so
    if (threadIdx.x < p) {
        __threadfence_system();
        red_add_release_sys(P.flags[threadIdx.x] + rs_done_index(P, per, npanels) + me, 1);
    }
}

// ---------------------------------------------------------------------------------------------- the kernel
// kPair: the CTAs 2i and 2i+1 form a cluster and share 256 x 256 tiles (see the head of the file).  A pair walks the tile
// order in units of two m tiles: the tile coordinates are computed on a grid of m_tiles / 2 row blocks and CTA r of the pair
// takes row block 2 * mp + r.  Everything per row block (AG readiness, RS delivery counters, the epilogue) stays as it is.
template <bool kPair>
__device__ __forceinline__ void tp_gemm_body(const TpGemmParams &P, SharedStorage &S)
{
    constexpr int kSt = kPair ? kStagesPair : kStages;
    constexpr uint32_t kStB = kPair ? kStageBytesPair : kStageBytes;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int m_tiles = P.M / BM, n_tiles = P.N / BN, k_iters = P.K / BK;
    const int total_tiles = m_tiles * n_tiles;
    const int pw = panel_width(P, n_tiles), npanels = (n_tiles + pw - 1) / pw;
    volatile uint32_t *fail = &S.fail;
    const uint32_t cta_r = kPair ? cluster_ctarank() : 0u;   // 0: leader of the pair (issues the MMAs)
    // work units of the tile loops: tiles for single CTAs, pairs of tiles (same n tile, m tiles 2 mp and 2 mp + 1) for pairs
    const int unit_first = kPair ? (int)blockIdx.x / 2 : (int)blockIdx.x;
    const int unit_step = kPair ? P.n_gemm_ctas / 2 : P.n_gemm_ctas;
    const int units = kPair ? total_tiles / 2 : total_tiles;
    const int um_tiles = kPair ? m_tiles / 2 : m_tiles;
    auto unit_coords = [&](int t, int &mt, int &nt, int &panel) {
        tile_coords(P, t, n_tiles, um_tiles, pw, mt, nt, panel);
        if (kPair) mt = 2 * mt + (int)cta_r;
    };

    if (threadIdx.x == 0) {
        S.fail = 0;
        S.gemm_done = 0;
        S.early_count = 0;
        for (int i = 0; i < kSt; ++i) { mbar_init(&S.full_bar[i], 1); mbar_init(&S.empty_bar[i], 1); }
        // pair: the epilogue threads of both CTAs release an accumulator on the leader's barrier
        for (int i = 0; i < 2; ++i) { mbar_init(&S.tmem_full[i], 1); mbar_init(&S.tmem_empty[i], kPair ? 256 : 128); }
        for (int i = 0; i < kCommDepth; ++i) mbar_init(&S.comm_bar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if ((int)blockIdx.x >= P.n_gemm_ctas) {  // data-movement CTA (AG): one thread drives bulk asynchronous copies
        comm_role_ag(P, S, blockIdx.x - P.n_gemm_ctas, gridDim.x - P.n_gemm_ctas);
        if (threadIdx.x == 0) bulk_wait_all<0>();
        return;
    }
    if (warp == 1) {  // TMEM allocation by one full warp (pair: by one warp of each CTA, all 512 columns, so both get base 0)
        if (kPair) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    // pair: the other CTA's barriers are initialised and its TMEM is allocated before anything of mine reaches them
    if (kPair) cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = S.tmem_base;
    const uint64_t deadline = global_timer_ns() + P.timeout_ns;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            uint32_t it = 0;
            const uint64_t *chunk_ready = P.mode == TP_MODE_AG ? P.flags[P.rank] + 2 * P.nranks : nullptr;
            // pair: the bytes of both CTAs' loads are counted on the leader's barrier, which the leader arms for both
            for (int t = unit_first; t < units && !*fail; t += unit_step) {
                int mt, nt, panel;
                unit_coords(t, mt, nt, panel);
                const CUtensorMap *amap = &P.tmA;
                int arow = mt * BM;
                if (chunk_ready) {
                    const int per_r = m_tiles / P.nranks;
                    if (mt / per_r == P.rank) {  // my own rows come straight from the caller's shard: nothing to wait for
                        amap = &P.tmX;
                        arow = (mt - P.rank * per_r) * BM;
                    } else {  // a peer's rows have to be in local memory (pulled by the data-movement CTAs)
                        if (!wait_word_ge(chunk_ready + mt, P.epoch, false, deadline, fail)) { report(P, *fail, 600 + mt); break; }
                        fence_proxy_async();
                    }
                }
                for (int k = 0; k < k_iters; ++k, ++it) {
                    uint32_t s = it % kSt, ph = (it / kSt) & 1;
                    if (!mbar_wait_t<kPair>(&S.empty_bar[s], ph ^ 1, fail)) { report(P, *fail, 700); break; }
                    uint8_t *sa = S.tiles + (size_t)s * kStB, *sb = sa + kABytes;
                    if (kPair) {
                        if (cta_r == 0) mbar_expect_tx(&S.full_bar[s], 2 * kStageBytesPair);
                        const uint32_t full_leader = mapa_u32(smem_u32(&S.full_bar[s]), 0);
                        tma_load_2d_pair(sa, amap, full_leader, k * BK, arow);
                        tma_load_2d_pair(sb, &P.tmB, full_leader, k * BK, nt * BN + (int)cta_r * (BN / 2));  // my half of the B rows
                    } else {
                        mbar_expect_tx(&S.full_bar[s], kStageBytes);
                        tma_load_2d(sa, amap, &S.full_bar[s], k * BK, arow);
                        tma_load_2d(sb, &P.tmB, &S.full_bar[s], k * BK, nt * BN);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if ((!kPair || cta_r == 0) && elect_one()) {  // pair: only the leader issues; its MMAs read both CTAs' stages
            uint32_t it = 0, tile_i = 0;
            for (int t = unit_first; t < units && !*fail; t += unit_step, ++tile_i) {
                uint32_t buf = tile_i & 1, use = tile_i >> 1;
                if (!mbar_wait_t<kPair>(&S.tmem_empty[buf], (use & 1) ^ 1, fail)) { report(P, *fail, 800); break; }
                tc_fence_after();
                uint32_t d = tmem_base + buf * BN;
                for (int k = 0; k < k_iters; ++k, ++it) {
                    uint32_t s = it % kSt, ph = (it / kSt) & 1;
                    if (!mbar_wait_t<kPair>(&S.full_bar[s], ph, fail)) { report(P, *fail, 900); break; }
                    tc_fence_after();
                    uint8_t *sa = S.tiles + (size_t)s * kStB, *sb = sa + kABytes;
                    uint64_t da = make_smem_desc(sa), db = make_smem_desc(sb);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // advance 16 bf16 = 32 bytes along K inside the 128-byte swizzle atom: +2 in 16-byte units
                        if (kPair) umma_pair(d, da + (uint64_t)(2 * kk), db + (uint64_t)(2 * kk), (k | kk) != 0);
                        else umma(d, da + (uint64_t)(2 * kk), db + (uint64_t)(2 * kk), (k | kk) != 0);
                    }
                    // frees the stage (pair: in both CTAs) when the MMAs that read it are done
                    if (kPair) umma_commit_pair(&S.empty_bar[s]); else umma_commit(&S.empty_bar[s]);
                }
                // accumulator complete (pair: each CTA's epilogue waits on its own barrier)
                if (kPair) umma_commit_pair(&S.tmem_full[buf]); else umma_commit(&S.tmem_full[buf]);
            }
        }
    } else if (warp >= 2 && warp < 6) {
        // ------------------------------------------------------------------ epilogue: TMEM -> registers -> bf16 -> global
        const int q4 = warp & 3;  // a warp may only touch the TMEM lane quarter given by its index modulo 4
        uint32_t tile_i = 0, owner_ok = 0;
        const int per = P.nranks > 0 ? m_tiles / P.nranks : m_tiles;
        for (int t = unit_first; t < units && !*fail; t += unit_step, ++tile_i) {
            int mt, nt, panel;
            unit_coords(t, mt, nt, panel);
            uint32_t buf = tile_i & 1, use = tile_i >> 1;
            if (!mbar_wait_t<kPair>(&S.tmem_full[buf], use & 1, fail)) { report(P, *fail, 1000); break; }
            tc_fence_after();
            const int row = mt * BM + q4 * 32 + lane;
            __nv_bfloat16 *dst_row;
            int owner = 0;
            if (P.mode == TP_MODE_RS) {
                owner = mt / per;  // rows of block mt belong to rank `owner`; my partial goes to its slot number P.rank
                // the owner must have finished reducing the previous call's data in that slot (checked once per owner)
                if (!(owner_ok & (1u << owner))) {
                    if (!wait_word_ge(P.flags[P.rank] + rs_done_index(P, per, npanels) + owner, (P.epoch - 1) * (uint64_t)gridDim.x, true, deadline, fail)) { report(P, *fail, 1100 + owner); break; }
                    owner_ok |= 1u << owner;
                }
                const uint64_t slot_elems = (uint64_t)(P.M / P.nranks) * P.N;
                dst_row = P.partial[owner] + (uint64_t)P.rank * slot_elems + (uint64_t)(row - owner * per * BM) * P.N + (uint64_t)nt * BN;
            } else {
                dst_row = P.C + (uint64_t)row * P.ldc + (uint64_t)nt * BN;
            }
            // 64 columns at a time: TMEM -> registers -> bf16 -> this thread's 128-byte slot in shared memory -> one bulk
            // asynchronous store of the whole 128-byte row piece (full lines on HBM and on NVLink, nothing blocks)
            uint8_t *slot = S.epi + (size_t)(q4 * 32 + lane) * kEpiStride;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += kEpiCols) {
                uint32_t r0[32], r1[32];
                tmem_ld32(tmem_base + buf * BN + c0 + ((uint32_t)(q4 * 32) << 16), r0);
                tmem_ld32(tmem_base + buf * BN + c0 + 32 + ((uint32_t)(q4 * 32) << 16), r1);
                tmem_ld_wait();
                bulk_wait_read<0>();  // the previous piece has left the slot
                uint4 *o = (uint4 *)slot;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 w;
                    w.x = pack_bf16(r0[8 * v + 0], r0[8 * v + 1]);
                    w.y = pack_bf16(r0[8 * v + 2], r0[8 * v + 3]);
                    w.z = pack_bf16(r0[8 * v + 4], r0[8 * v + 5]);
                    w.w = pack_bf16(r0[8 * v + 6], r0[8 * v + 7]);
                    o[v] = w;
                }
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 w;
                    w.x = pack_bf16(r1[8 * v + 0], r1[8 * v + 1]);
                    w.y = pack_bf16(r1[8 * v + 2], r1[8 * v + 3]);
                    w.z = pack_bf16(r1[8 * v + 4], r1[8 * v + 5]);
                    w.w = pack_bf16(r1[8 * v + 6], r1[8 * v + 7]);
                    o[4 + v] = w;
                }
                fence_proxy_async_smem();
                bulk_s2g(dst_row + c0, slot, kEpiCols * 2);
                bulk_commit();
            }
            tc_fence_before();
            // 128 arrivals (pair: 256, on the leader's barrier) free the accumulator for the tile after next
            if (kPair) mbar_arrive_cluster(mapa_u32(smem_u32(&S.tmem_empty[buf]), 0)); else mbar_arrive(&S.tmem_empty[buf]);
            if (P.mode == TP_MODE_RS) {
                // the four epilogue warps finished their rows: one of them publishes the tile to the owner
                // (no fence per thread: 128 system-scope fences per tile cost more than the whole transfer; the completed
                // bulk stores are ordered before the barrier, and the one release below publishes them)
                bulk_wait_all<0>();  // this thread's row pieces are written
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    red_add_release_sys(P.flags[owner] + ((uint64_t)P.rank * per + (mt - owner * per)) * npanels + panel, 1);
                }
            }
        }
    }
    else if (P.mode == TP_MODE_RS) {
        // ------------------------------------------------------------------ spare warps: reduce what has already arrived
        reduce_early_rs(P, S, pw, npanels);
    }
    if (warp >= 2 && warp < 6) {
        bulk_wait_all<0>();  // every row piece of this thread has been written
        if (P.mode == TP_MODE_RS && warp == 2 && lane == 0) *(volatile uint32_t *)&S.gemm_done = 1;
    }
    tc_fence_before();
    __syncthreads();
    // pair: the leader's MMAs read my stages and write my TMEM, and its commits arrive on my barriers: neither CTA lets go of
    // its shared memory or TMEM before both are through (every wait above is bounded, so both get here)
    if (kPair) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        if (kPair) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (P.mode == TP_MODE_RS && !__syncthreads_or((int)*fail)) reduce_tail_rs(P, S, pw, npanels);
}

__global__ void __launch_bounds__(kThreads, 1) tp_gemm_kernel(const __grid_constant__ TpGemmParamsArray PA)
{
    extern __shared__ uint8_t smem_raw[];
    SharedStorage &S = *(SharedStorage *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    tp_gemm_body<false>(PA.r[blockIdx.y], S);
}

// Launched with clusters of two CTAs along x.
__global__ void __launch_bounds__(kThreads, 1) tp_gemm_pair_kernel(const __grid_constant__ TpGemmParamsArray PA)
{
    extern __shared__ uint8_t smem_raw[];
    SharedStorage &S = *(SharedStorage *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    tp_gemm_body<true>(PA.r[blockIdx.y], S);
}

HcclResult encode_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    const DriverApi &d = driver_api();
    if (!d.ok || !d.TensorMapEncodeTiled) return HCCL_E_DRV;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = d.TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        HLOG_ERROR("cuTensorMapEncodeTiled failed: %s", cu_err(r));
        return HCCL_E_DRV;
    }
    return HCCL_SUCCESS;
}

}  // namespace

size_t tp_gemm_smem_bytes() { return sizeof(SharedStorage) + 1024; }

static std::atomic<uint64_t> g_launches[2];
void tp_gemm_launch_counts(uint64_t *single, uint64_t *pair)
{
    *single = g_launches[0].load();
    *pair = g_launches[1].load();
}

HcclResult launch_tp_gemm(TpGemmParams *P, const void *const *A, const void *const *B, int nlocal, int n_comm_ctas, void *stream)
{
    if (nlocal < 1 || nlocal > kTpMaxLocal) return HCCL_E_PARA;
    const TpGemmParams &P0 = P[0];
    if (P0.M % BM || P0.N % BN || P0.K % BK || P0.M <= 0 || P0.N <= 0 || P0.K <= 0) {
        HLOG_ERROR("fused GEMM needs M %% %d == 0, N %% %d == 0, K %% %d == 0 (got %d x %d x %d)", BM, BN, BK, P0.M, P0.N, P0.K);
        return HCCL_E_PARA;
    }
    if (P0.mode != TP_MODE_PLAIN && P0.nranks > 1 && (P0.M / BM) % P0.nranks) {
        HLOG_ERROR("fused GEMM needs the %d row blocks to divide evenly over %d ranks", P0.M / BM, P0.nranks);
        return HCCL_E_PARA;
    }
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // AG: a few CTAs only move data (bulk asynchronous copies); RS needs none (reduce tail on every CTA)
    if (P0.mode != TP_MODE_AG || P0.nranks == 1) n_comm_ctas = 0;  // a single rank has nothing to move: every CTA computes
    else if (n_comm_ctas < 1) n_comm_ctas = 1;
    int per_rank = sms / nlocal;  // all CTAs of all local ranks must be resident together
    if (n_comm_ctas > per_rank / 4) n_comm_ctas = n_comm_ctas ? std::max(1, per_rank / 4) : 0;
    if (n_comm_ctas > kMaxCommCtas) n_comm_ctas = kMaxCommCtas;
    // with communication every rank must run the same grid (completion counters count CTAs)
    int total = (P0.M / BM) * (P0.N / BN);
    // pair variant (clusters of two CTAs on 256 x 256 tiles): every rank's rows must come in pairs of 128-row blocks.  The
    // choice depends on the shape and the environment only, so every rank makes the same one.
    const int rows_per_rank = P0.mode == TP_MODE_PLAIN || P0.nranks < 1 ? P0.M : P0.M / P0.nranks;
    const bool pair = env_config().tp_gemm_pair && rows_per_rank % (2 * BM) == 0 && per_rank >= 4;
    if (pair) {
        // clusters that can be resident together (a cluster needs both of its SMs inside one GPC): asked once per device
        static std::mutex occ_mu;
        static int occ_clusters[64] = {0};
        int max_clusters = 0;
        {
            std::lock_guard<std::mutex> lk(occ_mu);
            if (dev >= 0 && dev < 64 && occ_clusters[dev] > 0) max_clusters = occ_clusters[dev];
            else {
                cudaFuncSetAttribute((const void *)tp_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tp_gemm_smem_bytes());
                cudaLaunchConfig_t q;
                memset(&q, 0, sizeof(q));
                q.gridDim = dim3((unsigned)(sms & ~1)); q.blockDim = dim3(kThreads); q.dynamicSmemBytes = tp_gemm_smem_bytes();
                cudaLaunchAttribute qa[1];
                qa[0].id = cudaLaunchAttributeClusterDimension;
                qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
                q.attrs = qa; q.numAttrs = 1;
                cudaError_t oe = cudaOccupancyMaxActiveClusters(&max_clusters, (const void *)tp_gemm_pair_kernel, &q);
                if (oe != cudaSuccess || max_clusters < 2) { HLOG_ERROR("cluster occupancy query failed: %s", cudaGetErrorString(oe)); return HCCL_E_RUNTIME; }
                if (dev >= 0 && dev < 64) occ_clusters[dev] = max_clusters;
            }
        }
        per_rank = std::min(per_rank, 2 * max_clusters / nlocal);
        per_rank &= ~1;
        if (n_comm_ctas) n_comm_ctas = std::min((n_comm_ctas + 1) & ~1, std::max(2, (per_rank / 4) & ~1));
    }
    int n_gemm = P0.mode == TP_MODE_PLAIN ? std::min(total, per_rank) : per_rank - n_comm_ctas;
    TpGemmParamsArray arr;
    memset(&arr, 0, sizeof(arr));
    for (int i = 0; i < nlocal; ++i) {
        if ((((uintptr_t)A[i]) | ((uintptr_t)B[i])) & 15) return HCCL_E_PARA;
        P[i].n_gemm_ctas = n_gemm;
        CHK_RET(encode_2d(&P[i].tmA, A[i], (uint64_t)P[i].M, (uint64_t)P[i].K, BM));
        if (P[i].mode == TP_MODE_AG) {
            if (((uintptr_t)P[i].x_shard) & 15) return HCCL_E_PARA;
            CHK_RET(encode_2d(&P[i].tmX, P[i].x_shard, (uint64_t)(P[i].M / P[i].nranks), (uint64_t)P[i].K, BM));
        }
        CHK_RET(encode_2d(&P[i].tmB, B[i], (uint64_t)P[i].N, (uint64_t)P[i].K, pair ? BN / 2 : BN));  // pair: a CTA loads half of the tile's B rows
        arr.r[i] = P[i];
    }
    // the opt-in to large dynamic shared memory belongs to the (device, function) pair: once per device, not per process
    // (a process may drive several GPUs, one thread each)
    static std::mutex attr_mu;
    static bool attr_set[2][64] = {{false}};
    size_t smem = tp_gemm_smem_bytes();
    const void *fn = pair ? (const void *)tp_gemm_pair_kernel : (const void *)tp_gemm_kernel;
    {
        std::lock_guard<std::mutex> lk(attr_mu);
        if (dev < 0 || dev >= 64 || !attr_set[pair][dev]) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) { HLOG_ERROR("cannot raise dynamic shared memory to %zu: %s", smem, cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
            if (dev >= 0 && dev < 64) attr_set[pair][dev] = true;
        }
    }
    dim3 grid((unsigned)(n_gemm + n_comm_ctas), (unsigned)nlocal), block(kThreads);
    // AG and RS mode make CTAs of one rank wait on each other (GEMM CTAs on the data-movement CTAs, the reduce tail on the
    // other CTAs' tiles): a cooperative launch guarantees that all of them are resident together even when another kernel
    // shares the GPU.  The plain GEMM has no such dependency.
    // (a single rank in AG mode has no data-movement CTAs and waits for nobody)
    const bool coop = nlocal > 1 || P0.mode == TP_MODE_RS || (P0.mode == TP_MODE_AG && P0.nranks > 1);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attrs[2];
    unsigned na = 0;
    if (pair) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 2; attrs[na].val.clusterDim.y = 1; attrs[na].val.clusterDim.z = 1;
        ++na;
    }
    if (coop) {
        attrs[na].id = cudaLaunchAttributeCooperative;
        attrs[na].val.cooperative = 1;
        ++na;
    }
    cfg.attrs = attrs; cfg.numAttrs = na;
    void *kargs[] = {(void *)&arr};
    cudaError_t e = cudaLaunchKernelExC(&cfg, fn, kargs);
    if (e != cudaSuccess) { HLOG_ERROR("fused GEMM launch failed (%s%s): %s", pair ? "pair " : "", coop ? "cooperative" : "plain", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    g_launches[pair ? 1 : 0]++;
    return HCCL_SUCCESS;
}

}  // namespace hcclb

// ---------------------------------------------------------------------------------------------- no-allocation entry point
// See kernels/fused/tp_gemm_noalloc.h.  The scratch that the row-parallel kernel normally gets from the communicator's
// symmetric heap (completion counters followed by the bf16 receive slot) lives in this file-scope device array instead.
namespace {
constexpr size_t kNoAllocFlagBytes = 64 * 1024;
constexpr size_t kNoAllocScratchBytes = kNoAllocFlagBytes + HCCLB200_NOALLOC_MAX_OUT_ELEMS * 2;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// The last 64 bytes of the counter area hold the failure word: the first bounded wait of a call that runs out leaves its
// code there (cleared with the counters at the next call).
constexpr size_t kNoAllocFailOffset = kNoAllocFlagBytes - 64;
struct NoAllocDeviceState {
    unsigned char *scratch = nullptr;  // device address of g_noalloc_scratch on that device
};
NoAllocDeviceState g_noalloc_state[64];
std::mutex g_noalloc_mu;  // first calls from several threads set the table up one at a time
}  // namespace

extern "C" int hcclb200_matmul_reduce_noalloc(const void *h, const void *w, void *out, int M, int N, int K, void *stream)
{
    using namespace hcclb;
    if (!h || !w || !out) return HCCL_E_PTR;
    if (M <= 0 || N <= 0 || K <= 0 || M % BM || N % BN || K % BK) return HCCL_E_PARA;
    if ((uint64_t)M * (uint64_t)N > HCCLB200_NOALLOC_MAX_OUT_ELEMS) {
        HLOG_ERROR("hcclb200_matmul_reduce_noalloc: M x N = %llu exceeds the built-in scratch of %llu elements",
                   (unsigned long long)M * N, (unsigned long long)HCCLB200_NOALLOC_MAX_OUT_ELEMS);
        return HCCL_E_MEMORY;
    }
    if (tp_flag_words(M, 1) * 8 > kNoAllocFailOffset) return HCCL_E_MEMORY;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HCCL_E_RUNTIME;
    NoAllocDeviceState &st = g_noalloc_state[dev];
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!st.scratch) {
        // first call on this device: in host code the array's name is only a stand-in, the kernel needs the device address
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            HLOG_ERROR("cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
            return HCCL_E_RUNTIME;
        }
        st.scratch = (unsigned char *)p;
    }
    // the array keeps the previous call's contents and calls may differ in shape: the completion counters must start at
    // zero for every call (the receive slot needs no clearing, it is rewritten before it is read)
    if (cudaMemsetAsync(st.scratch, 0, kNoAllocFlagBytes, (cudaStream_t)stream) != cudaSuccess) return HCCL_E_RUNTIME;
    TpGemmParams P;
    memset(&P, 0, sizeof(P));
    P.mode = TP_MODE_RS; P.M = M; P.N = N; P.K = K; P.rank = 0; P.nranks = 1;
    P.epoch = 1;
    P.timeout_ns = 10000000000ull;
    P.out = (__nv_bfloat16 *)out;
    P.flags[0] = (uint64_t *)st.scratch;
    P.partial[0] = (__nv_bfloat16 *)(st.scratch + kNoAllocFlagBytes);
    P.fail_word = (uint32_t *)(st.scratch + kNoAllocFailOffset);
    const void *a[1] = {h}, *b[1] = {w};
    return launch_tp_gemm(&P, a, b, 1, 0, stream);
}

extern "C" int hcclb200_matmul_reduce_noalloc_status(void *stream)
{
    using namespace hcclb;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HCCL_E_RUNTIME;
    unsigned char *scratch;
    {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        scratch = g_noalloc_state[dev].scratch;
    }
    if (!scratch) return HCCL_SUCCESS;  // nothing has run on this device yet
    uint32_t code = 0;
    if (cudaMemcpyAsync(&code, scratch + kNoAllocFailOffset, sizeof(code), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess ||
        cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess)
        return HCCL_E_RUNTIME;
    return (int)code;
}
