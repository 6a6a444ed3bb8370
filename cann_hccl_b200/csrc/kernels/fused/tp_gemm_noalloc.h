/*
 * hcclb200_matmul_reduce_noalloc — the row-parallel "GEMM + reduce" kernel for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference library (HCCL always takes its scratch from the
 * communicator's CCL buffers).  It exists for code that runs where device allocation is forbidden or unsafe:
 * a plugin called from inside another framework's stream-ordered allocator, a real-time loop that has to keep the
 * driver's allocation lock out of its path, a process that has handed all free memory to a memory pool and would fail
 * a cudaMalloc, or a host without a communicator (and therefore without the communicator's symmetric heap).
 *
 *   out[M, N] (bf16) = h[M, K] (bf16) * w[N, K]^T (bf16), fp32 accumulation,
 *
 * computed by the same sm_100a kernel and the same path as HcclB200MatmulReduceScatter on a one-rank communicator:
 * the epilogue writes bf16 partial tiles into a receive slot, completion counters are bumped, and the reduce tail sums
 * the (single) slot into `out`.  The receive slot and the counters are the kernel's scratch memory.  Here they live
 * in a file-scope `static __device__` array inside the library instead of in memory allocated at run time:
 *
 *   - the array holds 64 KiB of counters and HCCLB200_NOALLOC_MAX_OUT_ELEMS bf16 values (4 MiB + 64 KiB in total);
 *     every GPU that loads the library carries it until the process exits;
 *   - M * N must not exceed HCCLB200_NOALLOC_MAX_OUT_ELEMS; larger problems are rejected with HCCL_E_MEMORY (3) and
 *     nothing is launched.  M % 128 == 0, N % 256 == 0, K % 64 == 0, pointers 16-byte aligned (HCCL_E_PARA otherwise).
 *   - the call performs no cudaMalloc / cudaFree and calls no allocating library routine; the caller passes inputs and
 *     output only;
 *   - the first call on a device does the set-up for that device (it asks the runtime for the array's device address
 *     with cudaGetSymbolAddress).  Make that first call outside of any stream capture;
 *   - all calls on a device share the one array, and it keeps what the previous call left in it: every call therefore
 *     clears the counters on `stream` before its kernel (a 64 KiB cudaMemsetAsync); the receive slot needs no clearing
 *     because it is fully rewritten before it is read.  Two calls that overlap on the GPU (different streams, no ordering
 *     between them) race on the array: keep the calls of one device in stream order.
 *
 * Returns an HcclResult value as int (0 = success).  That value covers argument checks and the launch only.  The kernel's
 * own waits are bounded; if one runs out, `out` is incomplete and the kernel leaves its code (HCCL_E_TIMEOUT) in a word
 * inside the same static array.  hcclb200_matmul_reduce_noalloc_status(stream) waits for `stream`, reads that word with a
 * 4-byte copy into a stack variable (no allocation either) and returns it: 0 when the newest call on this device ran to
 * the end.  The word is cleared together with the counters at the start of the next call.
 * First calls on a device may come from several threads at once: the set-up is serialised inside the library.
 */
#ifndef HCCLB200_TP_GEMM_NOALLOC_H_
#define HCCLB200_TP_GEMM_NOALLOC_H_

#define HCCLB200_NOALLOC_MAX_OUT_ELEMS (2ull * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif
int hcclb200_matmul_reduce_noalloc(const void *h, const void *w, void *out, int M, int N, int K, void *stream);
int hcclb200_matmul_reduce_noalloc_status(void *stream);
#ifdef __cplusplus
}
#endif
#endif
