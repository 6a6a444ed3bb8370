/*
 * Extensions of the HCCL-compatible API that exist only in the B200 library:
 * the rooted Gather and the count-matrix AlltoAllVC that HCCL keeps internal, all-local communicators
 * (every rank a virtual rank of one GPU or a CPU thread; used for single-GPU validation of the multi-rank
 * kernels), forced-algorithm collectives, symmetric memory, selector / statistics / trace queries, and the
 * fused tensor-parallel and MoE kernels.
 */
#ifndef HCCL_B200_H_
#define HCCL_B200_H_
#include <sys/types.h>
#include "hccl.h"
#ifdef __cplusplus
extern "C" {
#endif

/* Collective kinds and algorithm ids accepted by HcclB200Collective / HcclB200Select. */
enum { HCCL_B200_ALLREDUCE = 0, HCCL_B200_BROADCAST, HCCL_B200_REDUCE_SCATTER, HCCL_B200_REDUCE_SCATTER_V,
       HCCL_B200_SCATTER, HCCL_B200_ALLGATHER, HCCL_B200_ALLGATHER_V, HCCL_B200_BARRIER, HCCL_B200_ALLTOALL,
       HCCL_B200_ALLTOALLV, HCCL_B200_ALLTOALLVC, HCCL_B200_REDUCE, HCCL_B200_GATHER };
enum { HCCL_B200_ALGO_AUTO = 0, HCCL_B200_ALGO_MESH, HCCL_B200_ALGO_MESH_ONESHOT, HCCL_B200_ALGO_RING,
       HCCL_B200_ALGO_RHD, HCCL_B200_ALGO_PAIRWISE, HCCL_B200_ALGO_STAR, HCCL_B200_ALGO_TREE, HCCL_B200_ALGO_NVLS,
       HCCL_B200_ALGO_NVLS_ONESHOT, HCCL_B200_ALGO_SINGLE, HCCL_B200_ALGO_MESH_PIPE, HCCL_B200_ALGO_NVLS_PIPE, HCCL_B200_ALGO_NVLS_ZEROCOPY, HCCL_B200_ALGO_LL, HCCL_B200_ALGO_MESH_ZEROCOPY, HCCL_B200_ALGO_DIRECT };

typedef struct HcclB200OpDef {
    int32_t coll;       /* HCCL_B200_* collective */
    int32_t algo;       /* HCCL_B200_ALGO_*, AUTO lets the selector decide */
    int32_t nchan;      /* CTAs per rank, 0 = selector */
    int32_t dataType;   /* HcclDataType */
    int32_t op;         /* HcclReduceOp */
    int32_t root;
    uint64_t count;     /* per-API count (see hccl.h) */
    const uint64_t *counts, *displs;                       /* AllGatherV / ReduceScatterV, nRanks entries */
    const uint64_t *sendCounts, *sdispls, *recvCounts, *rdispls; /* AlltoAllV: [local ranks][nRanks] */
} HcclB200Op;

/* Rooted gather: root's recvBuf receives nRanks blocks of sendCount elements in rank order. */
extern HcclResult HcclGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, uint32_t root,
                             HcclComm comm, aclrtStream stream);
/* AlltoAll with the full nRanks x nRanks send-count matrix (row i = counts rank i sends), blocks packed in rank order. */
extern HcclResult HcclAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType,
                                 const void *recvBuf, HcclDataType recvType, HcclComm comm, aclrtStream stream);

/* All ranks in this process: transport 0 = host memory + threads, 1 = virtual ranks on `device`. */
extern HcclResult HcclB200CommInitLocal(uint32_t nRanks, int transport, int device, const HcclCommConfig *config,
                                        HcclComm *comm);
/* Generic collective entry; sendBufs / recvBufs hold one pointer per local rank. */
extern HcclResult HcclB200Collective(HcclComm comm, const HcclB200Op *op, void *const *sendBufs, void *const *recvBufs,
                                     aclrtStream stream);
/* hccl_test-style loop issued from C: `iters` back-to-back collectives; call i shifts every buffer by
 * (i % nwin) * strideBytes so that successive calls touch different memory. */
extern HcclResult HcclB200Repeat(HcclComm comm, const HcclB200Op *op, void *const *sendBufs, void *const *recvBufs, uint32_t iters,
                                 uint64_t strideBytes, uint32_t nwin, aclrtStream stream);
/* The measured baseline: ncclAllReduce issued the same way on the NCCL communicator that carries Send/Recv. */
extern HcclResult HcclB200NcclAllReduceRepeat(HcclComm comm, void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType,
                                              HcclReduceOp op, uint32_t iters, uint64_t strideBytes, uint32_t nwin, aclrtStream stream);
extern HcclResult HcclB200LocalSendRecv(HcclComm comm, uint32_t src, uint32_t dst, const void *sendBuf, void *recvBuf,
                                        uint64_t count, HcclDataType dataType, aclrtStream stream);
/* Wait for the stream and return the status the kernels left (HCCL_E_TIMEOUT, HCCL_E_SUSPENDING, ...). */
extern HcclResult HcclB200StreamSync(HcclComm comm, aclrtStream stream);

typedef struct HcclB200StatusDef {
    uint32_t code, step; int32_t peer; uint32_t chan;
    uint64_t expected, seen, seq, head, tail;
} HcclB200Status;
/* ---- MoE expert-parallel dispatch / combine (kernels/moe_a2a.cu); bf16 rows, int32 expert ids, fp32 gates ---- */
/* hist[e] = pairs routed to expert e, pos[i] = arrival index of pair i inside its expert group. */
extern HcclResult HcclB200MoeCount(const int32_t *topkIdx, int64_t nPairs, int32_t nExperts, int32_t *hist, int32_t *pos, aclrtStream stream);
/* From the all-gathered histograms counts[nRanks][nExperts]: base[e] (first receive row of this rank's block for expert e on
 * its owner), this rank's expertOffsets[nExperts/nRanks + 1], recvRows, and overflow = 1 when recvRows > capacityRows. */
extern HcclResult HcclB200MoeOffsets(const int32_t *counts, int32_t nRanks, int32_t nExperts, int32_t rank, int32_t *base,
                                     int32_t *expertOffsets, int32_t *recvRows, int64_t capacityRows, int32_t *overflow, aclrtStream stream);
/* Store every (token, k) row into the owner's receive buffer (recvPeers[q] = rank q's buffer); records dstRow[i]. */
extern HcclResult HcclB200MoeDispatch(const void *x, const int32_t *topkIdx, const int32_t *pos, const int32_t *base, int64_t tokens,
                                      int32_t topk, int32_t hidden, int32_t nExperts, int32_t nRanks, int32_t rank, int32_t pairwise,
                                      void *const *recvPeers, int32_t *dstRow, int64_t capacityRows, aclrtStream stream);
/* out[t] = sum_k gates[t,k] * yPeers[owner][dstRow[t,k]] : the gate-weighted combine happens while the rows are received. */
extern HcclResult HcclB200MoeCombine(void *const *yPeers, const int32_t *topkIdx, const float *gates, const int32_t *dstRow, int64_t tokens,
                                     int32_t topk, int32_t hidden, int32_t nExperts, int32_t nRanks, int32_t rank, int32_t pairwise, void *out,
                                     int64_t capacityRows, aclrtStream stream);
/* ---- fused tensor-parallel kernels (tcgen05 GEMM + NVLink transfer in one sm_100a kernel); bf16, weights [N, K] ---- */
/* C[M,N] = A[M,K] * B[N,K]^T (no communication). M % 128 == 0, N % 256 == 0, K % 64 == 0. */
extern HcclResult HcclB200GemmBf16(const void *A, const void *B, void *C, int32_t M, int32_t N, int32_t K, aclrtStream stream);
/* Launches of the fused GEMM kernels in this process so far: *single on one CTA per tile (tcgen05 cta_group::1), *pair on
 * clusters of two CTAs per 256 x 256 tile (cta_group::2; HCCL_TP_GEMM_PAIR, shapes whose rows per rank are a multiple of 256). */
extern HcclResult HcclB200GemmLaunchCounts(uint64_t *single, uint64_t *pair);
/* Column-parallel layer: outs = all_gather_rows(xShards [M/p, K]) * weights[N, K]^T -> [M, N].  One pointer per local rank. */
extern HcclResult HcclB200AllGatherMatmul(HcclComm comm, void *const *xShards, void *const *weights, void *const *outs, int32_t M,
                                          int32_t N, int32_t K, aclrtStream stream);
/* Row-parallel layer: outs [M/p, N] = reduce_scatter_rows(inputs [M, K] * weights[N, K]^T). */
extern HcclResult HcclB200MatmulReduceScatter(HcclComm comm, void *const *inputs, void *const *weights, void *const *outs, int32_t M,
                                              int32_t N, int32_t K, aclrtStream stream);
/* In-kernel timestamps of the newest executor launch (needs HCCL_KERNEL_TRACE=1 at communicator creation):
 * out[0] = kernel start (globaltimer ns), then per step {after wait, after data movement, after signal}. */
extern HcclResult HcclB200GetKernelTrace(HcclComm comm, uint32_t localRank, uint64_t *out, size_t capWords, int32_t *nsteps);
/* Diagnostic: local rank waits (bounded by timeoutMs) for a flag nothing sets; returns HCCL_E_TIMEOUT and fills the
 * status block.  The communicator must be resumed afterwards.  Proves that a starved wait ends and leaves the
 * context usable. */
extern HcclResult HcclB200WaitProbe(HcclComm comm, uint32_t localRank, double timeoutMs, aclrtStream stream);
extern HcclResult HcclB200GetStatus(HcclComm comm, uint32_t localRank, HcclB200Status *status);
/* Human readable decoding of a status block (role of the reference's task exception handler). */
extern HcclResult HcclB200DescribeStatus(HcclComm comm, uint32_t localRank, char *text, size_t cap);

extern HcclResult HcclB200Select(HcclComm comm, int32_t coll, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                                 int32_t *algo, int32_t *nchan, double *estimateUs);
extern HcclResult HcclB200GetStatsJson(HcclComm comm, char *json, size_t cap);
extern HcclResult HcclB200GetTraceJson(HcclComm comm, char *json, size_t cap);
extern HcclResult HcclB200Calibrate(HcclComm comm, aclrtStream stream);
extern HcclResult HcclB200SetCostModel(HcclComm comm, double alphaUs, double betaGBps, double nvlsGBps, double gammaGBps,
                                       double launchUs);
extern const char *HcclB200GetLastError(void);
extern const char *HcclB200AlgoName(int32_t algo);
extern HcclResult HcclB200HasNvls(HcclComm comm, int32_t *has);
extern HcclResult HcclB200GetLocalRankNum(HcclComm comm, uint32_t *n);

/* Symmetric memory: same-size allocation on every rank, peers mapped.  localPtrs gets one pointer per local rank. */
extern HcclResult HcclB200MemAlloc(HcclComm comm, size_t bytes, void **localPtrs, int32_t *handle);
/* Registers memory the caller owns (one pointer per local rank, `bytes` each) as a symmetric allocation: peers map it and
 * zero-copy collectives, put/get and the fused kernels accept it like memory from HcclB200MemAlloc.  Collective.  With one
 * rank per GPU, drvHandles[0] is the driver allocation handle behind the pointer (created exportable as a POSIX file
 * descriptor; whole allocation, handleOffset 0); with virtual ranks in one process drvHandles may be NULL.
 * HcclB200MemFree ends the registration and leaves the memory alone.  This is what HcclCommActivateCommMemory calls. */
extern HcclResult HcclB200MemAdopt(HcclComm comm, void *const *localPtrs, size_t bytes, const uint64_t *drvHandles, size_t handleOffset,
                                   int32_t *handle);
extern HcclResult HcclB200MemFree(HcclComm comm, int32_t handle);
/* Allocator hooks for frameworks with pluggable device allocators (torch.cuda.memory.CUDAPluggableAllocator + MemPool):
 * after HcclB200PoolBind(comm), hcclb200_torch_malloc / hcclb200_torch_free serve the framework's pool from registered
 * symmetric memory of that communicator, so collectives on tensors of the pool run zero-copy.  Allocation is collective
 * (same sizes in the same order on every rank); freed blocks are reused, and released when the pool is unbound
 * (HcclB200PoolBind(NULL), collective) or the communicator is destroyed. */
extern HcclResult HcclB200PoolBind(HcclComm comm);
extern void *hcclb200_torch_malloc(ssize_t size, int device, void *stream);
extern void hcclb200_torch_free(void *ptr, ssize_t size, int device, void *stream);
/* peerPtrs[local * nRanks + q] = rank q's copy as mapped for the local rank; mcPtrs[local] = multicast mapping or NULL. */
extern HcclResult HcclB200MemQuery(HcclComm comm, int32_t handle, void **peerPtrs, void **mcPtrs, size_t *bytes);
/* One-sided transfers on symmetric memory (role of the reference's one_sided_service interface,
 * communicator/impl/one_sided_service/): stream-ordered copy between a local buffer and `bytes` at `offset` inside rank
 * `peer`'s copy of allocation `handle`.  Only the calling rank takes part; pair with HcclBarrier (or any collective) to
 * order against the peer's own accesses.  `localRank` selects the virtual rank on an all-local communicator, else 0. */
extern HcclResult HcclB200Put(HcclComm comm, uint32_t localRank, int32_t handle, uint32_t peer, size_t offset, const void *src,
                              size_t bytes, aclrtStream stream);
extern HcclResult HcclB200Get(HcclComm comm, uint32_t localRank, int32_t handle, uint32_t peer, size_t offset, void *dst,
                              size_t bytes, aclrtStream stream);
/* Topology of the communicator as JSON: ranks (host, pid, device), transport, NVLS, peer-access matrix of local devices. */
extern HcclResult HcclB200GetTopoJson(HcclComm comm, char *json, size_t cap);
/* Overflow check (role of the reference's TaskOverflow hookup): with HCCL_OVERFLOW_CHECK=1 every floating-point reduction
 * is followed by a scan of its output; *count = outputs that were Inf or NaN since the communicator was made. */
extern HcclResult HcclB200GetOverflowCount(HcclComm comm, uint64_t *count);
/* Offline lint of a schedule: lowers (coll, algo) for nRanks ranks and `count` elements and runs the static bounds check
 * that every plan passes before its first execution (operand ranges against staging / mailbox / caller buffer sizes, channel,
 * bank and rank fields).  skewStep >= 0 adds skewBytes to the destination offset of that step of rank 0 first, to show the
 * check firing.  message receives the plan name, or the first violation.  No communicator and no GPU needed. */
extern HcclResult HcclB200PlanCheck(int32_t coll, int32_t algo, uint32_t nRanks, uint64_t count, HcclDataType dataType, uint32_t nChannels,
                                    uint64_t stageHalfBytes, int32_t skewStep, int64_t skewBytes, char *message, size_t cap);
/* Static race detection of the plan of (collective, algorithm) for nRanks ranks and nChannels channels (CTAs) per rank: builds the
 * happens-before relation (program order per rank and channel + flag signal -> wait) and demands that conflicting accesses to
 * the staging, send and receive buffers are ordered by it; also reports waits that nothing satisfies and cycles.  inPlace != 0
 * folds each rank's send and receive buffer into one, the way the collective's in-place form lays them out.  dropWaitRank /
 * dropWaitStep >= 0 remove the wait of that step first (to see the checker find the hole; HCCL_E_PARA when the step has none).
 * message receives the plan's name, or the first finding. */
extern HcclResult HcclB200PlanRaceCheck(int32_t coll, int32_t algo, uint32_t nRanks, uint64_t count, HcclDataType dataType, uint32_t nChannels,
                                        uint32_t root, int32_t inPlace, int32_t dropWaitRank, int32_t dropWaitStep, char *message, size_t cap);
/* All-gather `len` bytes per rank over the bootstrap hub (control plane; not for bulk data). */
extern HcclResult HcclB200Exchange(HcclComm comm, const char *tag, const void *mine, size_t len, void *all);
/* Context handed to custom kernels (role of the reference's MC2 resource export, op_base.cc:3137-3284):
 * device array of per-local-rank contexts with peer staging / flag pointers, plus the next op sequence number. */
extern HcclResult HcclB200GetDeviceContext(HcclComm comm, void **devCtxArray, uint64_t *nextSeq);
extern HcclResult HcclB200ReloadEnv(void);
/* NVLink attributes of a GPU as JSON: ports, active links, links that end in an NVSwitch, NVLink generation, bandwidth per
 * link and direction, multicast capability.  Read from the management library (HCCL_NVML_LIB names another one). */
extern HcclResult HcclB200ProbeLinks(int32_t device, char *json, size_t cap);
/* Staged abort over every communicator of `device` (-1: all devices and CPU communicators), the role of the reference's
 * task-abort callback: stage 0 suspends (no new operations, waits in flight are told to end), stage 1 waits for the kernels
 * in flight to exit, stage 2 clears status blocks and counters; HcclCommResume (collective) makes the communicators usable
 * again.  Each communicator gets `timeoutSec` per stage (0 = no limit).  Returns 0 = done, 1 = failed, 2 = timed out. */
extern int32_t HcclB200TaskAbort(int32_t device, int32_t stage, uint32_t timeoutSec);

#ifdef __cplusplus
}
#endif
#endif
