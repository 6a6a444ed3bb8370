// Parametric AlltoAll(V/VC) kernel for sm_100a: see a2av.h.
//
// Every ordered pair of ranks (i -> j) is served by `lanes` independent streams.  Lane l of the pair moves its share of
// the block in rounds through two sub-slots of the receiver's staging half: the sending CTA on rank i copies a round into
// sub-slot r % 2 on rank j with bulk asynchronous copies (a peer store, no peer load) and publishes data flag r + 1; the
// receiving CTA on rank j copies the sub-slot to its place in the receive buffer and publishes ack flag r + 1, which
// frees the sub-slot for round r + 2.  Both sides derive the number of rounds from their own count (what i sends to j is
// what j expects from i), so nothing global is needed.  A CTA only ever waits for a CTA of another rank: no dependency
// inside a rank.  Waits are bounded; a CTA that gives up records the status block.
#include <cuda_runtime.h>
#include <mutex>
#include <set>
#include <utility>
#include "common/log.h"
#include "kernels/a2av.h"
#include "kernels/pipe_coll.cuh"

namespace hcclb {

namespace {

constexpr int kA2avThreads = 128;

__global__ void __launch_bounds__(kA2avThreads, 1) a2av_kernel(const RankCtx *ctxs, const A2avArgsArray args)
{
    using namespace pipe_detail;
    extern __shared__ __align__(128) uint8_t ring[];
    const A2avArgs &a = args.a[blockIdx.y];
    const int tid = threadIdx.x, b = blockIdx.x;
    __shared__ RankCtx s_ctx;
    __shared__ int s_fail, s_last;
    __shared__ const uint8_t *s_src[1];
    __shared__ uint8_t *s_dst[1];
    __shared__ uint64_t s_bytes[1];
    __shared__ __align__(8) uint64_t s_bar[kTmaDepth];
    {
        const uint64_t *gs = (const uint64_t *)&ctxs[blockIdx.y];
        for (int i = tid; i < (int)(sizeof(RankCtx) / 8); i += blockDim.x) ((uint64_t *)&s_ctx)[i] = gs[i];
    }
    if (tid == 0) {
        s_fail = 0;
        for (int i = 0; i < kTmaDepth; ++i) mbar_init(&s_bar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const RankCtx &c = s_ctx;
    const int me = c.rank, p = c.nranks, es = dtype_size(a.dtype), L = a.lanes;
    WaitCtx w;
    w.deadline = global_timer_ns() + c.timeout_ns;
    w.abort = c.abort;
    w.local_fail = c.exit_counter + 1;
    const uint64_t half_off = (a.seq & 1) * c.stage_half;
    const uint64_t base = a.seq << kSeqShift;
    uint32_t tma_g = 0;
    // CTA -> (direction, peer, lane)
    const int lane = b % L, peer = (b / L) % p, sending = b / (L * p) == 0;
    if (a.seq >= 2) {  // the peers must have left the op that used this staging half before
        if (tid < p && tid != me) {
            uint64_t seen;
            int rc = wait_flag_ge(c.flags[me] + done_index(tid), a.seq - 2, w, seen);
            if (rc) { report_failure(c, a.seq, rc, -1, tid, b, a.seq - 2, seen); s_fail = rc; }
        }
        __syncthreads();
    }
    // this lane's share [lo, hi) of the block exchanged with `peer` (bytes; 16-byte pieces)
    const uint64_t block = (sending ? a.send_counts[peer] : a.recv_counts[peer]) * (uint64_t)es;
    const uint64_t per = round_up_u64(ceil_div_u64(block, (uint64_t)L), 16);
    const uint64_t lo = per * lane < block ? per * lane : block, hi = lo + per < block ? lo + per : block;
    const uint64_t rounds = ceil_div_u64(hi - lo, a.sub_bytes);
    auto copy_one = [&](const uint8_t *src, uint8_t *dst, uint64_t bytes) {
        if (tid == 0) { s_src[0] = src; s_dst[0] = dst; s_bytes[0] = bytes; }
        __syncthreads();
        if (aligned16(src) && aligned16(dst) && (bytes & 15) == 0) {
            if (tid == 0 && !tma_copy_segments(ring, s_bar, tma_g, 1, s_src, s_dst, s_bytes)) {
                report_failure(c, a.seq, HCCL_E_TIMEOUT, -2, peer, b, 0, 0);
                s_fail = HCCL_E_TIMEOUT;
            }
        } else {
            pipe_copy_segments(s_src, s_dst, s_bytes, 1, es);
        }
        __syncthreads();
    };
    if (peer == me) {
        // the block a rank sends to itself: straight from the send buffer to the receive buffer (sending CTAs only)
        if (sending && hi > lo && !s_fail) copy_one(a.in + a.send_displs[me] * es + lo, a.out + a.recv_displs[me] * es + lo, hi - lo);
    } else {
        // slot of (source rank, lane) inside the receiver's staging half
        const int src_rank = sending ? me : peer, dst_rank = sending ? peer : me;
        uint8_t *slot = c.stage[dst_rank] + half_off + ((uint64_t)src_rank * L + lane) * 2 * a.sub_bytes;
        for (uint64_t r = 0; r < rounds && !s_fail; ++r) {
            const uint64_t off = lo + r * a.sub_bytes, nb = hi - off < a.sub_bytes ? hi - off : a.sub_bytes;
            uint8_t *sub = slot + (r & 1) * a.sub_bytes;
            if (sending) {
                if (r >= 2) {  // the receiver has emptied this sub-slot of round r - 2
                    if (tid == 0) {
                        uint64_t seen;
                        int rc = wait_flag_ge(c.flags[me] + flag_index(1, peer, lane), base + r - 1, w, seen);
                        if (rc) { report_failure(c, a.seq, rc, (int)r, peer, b, base + r - 1, seen); s_fail = rc; }
                    }
                    __syncthreads();
                    if (s_fail) break;
                }
                copy_one(a.in + a.send_displs[peer] * es + off, sub, nb);
                if (tid == 0 && !s_fail) st_release_sys(c.flags[peer] + flag_index(0, me, lane), base + r + 1);
            } else {
                if (tid == 0) {
                    uint64_t seen;
                    int rc = wait_flag_ge(c.flags[me] + flag_index(0, peer, lane), base + r + 1, w, seen);
                    if (rc) { report_failure(c, a.seq, rc, (int)r, peer, b, base + r + 1, seen); s_fail = rc; }
                }
                __syncthreads();
                if (s_fail) break;
                copy_one(sub, a.out + a.recv_displs[peer] * es + off, nb);
                if (tid == 0 && !s_fail) st_release_sys(c.flags[peer] + flag_index(1, me, lane), base + r + 1);
            }
        }
    }
    // completion: the last CTA of this rank tells every peer that this op no longer touches their memory
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        unsigned prev = atomicAdd(c.exit_counter, 1u);
        s_last = prev == gridDim.x - 1;
        if (s_last) *c.exit_counter = 0;
    }
    __syncthreads();
    if (s_last && !s_fail && *(volatile uint32_t *)(c.exit_counter + 1) == 0u) {
        if (tid < p && tid != me) st_release_sys(c.flags[tid] + done_index(me), a.seq);
        if (tid == 0) *c.dev_tail = a.seq;
    }
}

}  // namespace

HcclResult launch_a2av(const RankCtx *dev_ctx, const A2avArgs *args, int nlocal, int nranks, void *stream)
{
    if (nlocal < 1 || nlocal > kMaxRanks || nranks < 1 || nranks > kMaxRanks) return HCCL_E_PARA;
    const int L = args[0].lanes;
    if (L < 1 || L > kA2avMaxLanes || args[0].sub_bytes < 256 || (args[0].sub_bytes & 255)) return HCCL_E_PARA;
    static A2avArgsArray arr;  // too large for the stack of small threads; guarded by the communicator's operation lock per call
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    for (int i = 0; i < nlocal; ++i) arr.a[i] = args[i];
    {
        static std::set<int> done;
        int dev = 0;
        cudaGetDevice(&dev);
        if (!done.count(dev)) {
            cudaError_t e = cudaFuncSetAttribute(a2av_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPipeDynSmem);
            if (e != cudaSuccess) { HLOG_ERROR("cudaFuncSetAttribute(a2av kernel) failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
            done.insert(dev);
        }
    }
    dim3 grid((unsigned)(2 * nranks * L), (unsigned)nlocal), block(kA2avThreads);
    void *kargs[] = {(void *)&dev_ctx, (void *)&arr};
    // virtual ranks of one GPU wait on one another: their CTAs must be resident together
    cudaError_t e = nlocal > 1 ? cudaLaunchCooperativeKernel((const void *)a2av_kernel, grid, block, kargs, kPipeDynSmem, (cudaStream_t)stream)
                               : cudaLaunchKernel((const void *)a2av_kernel, grid, block, kargs, kPipeDynSmem, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        HLOG_ERROR("a2av kernel launch failed (grid %dx%d): %s", 2 * nranks * L, nlocal, cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace hcclb
