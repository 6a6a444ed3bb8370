"""Small, self-terminating workloads of each hot kernel, for profiling one kernel at a time on ONE GPU.

    python -m cann_hccl_b200.utils.profile_cases gemm        # tcgen05 GEMM 4096 x 3584 x 8192 (operands > L2)
    python -m cann_hccl_b200.utils.profile_cases gemm_rs     # same kernel in reduce-scatter mode on one rank
    python -m cann_hccl_b200.utils.profile_cases copy        # executor kernel, one rank, 64 MiB (the N=1 bench step)
    python -m cann_hccl_b200.utils.profile_cases allreduce   # executor kernel, two virtual ranks, two-shot 64 MiB fp32
    python -m cann_hccl_b200.utils.profile_cases ll          # LL AllReduce kernel, two virtual ranks, 256 KiB
    python -m cann_hccl_b200.utils.profile_cases moe         # MoE dispatch + combine, one rank, 2048 tokens x 7168

Each case runs a few launches and prints device-timed figures (CUDA events); under a profiler only the counters matter.
"""
import os
import sys

import torch

import cann_hccl_b200 as H
from cann_hccl_b200 import _lib as L
from cann_hccl_b200.parallel import fused_tp, moe


def _timed(fn, iters=3):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main(case):
    os.environ.setdefault("HCCL_EXEC_TIMEOUT_MS", "3000")
    torch.cuda.set_device(0)
    if case == "gemm":
        M, N, K = 4096, 3584, 8192
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = _timed(lambda: fused_tp.gemm(a, b, out=c))
        print("gemm %dx%dx%d: %.3f ms, %.0f TFLOP/s" % (M, N, K, ms, 2.0 * M * N * K / ms / 1e9))
    elif case == "gemm_rs":
        M, N, K = 4096, 4096, 3584
        comm = H.Communicator.init_root(1, H.Communicator.get_root_info(), 0, device=True)
        h = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        w = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        o = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = _timed(lambda: fused_tp.matmul_reduce_scatter(comm, h, w, out=o))
        assert comm.sync() == 0
        print("gemm_rs %dx%dx%d: %.3f ms, %.0f TFLOP/s" % (M, N, K, ms, 2.0 * M * N * K / ms / 1e9))
        comm.destroy()
    elif case == "copy":
        comm = H.Communicator.init_root(1, H.Communicator.get_root_info(), 0, device=True)
        n = 16 << 20
        x = torch.rand(4 * n, device="cuda")
        y = torch.empty_like(x)
        ms = _timed(lambda: comm.repeat(L.ALLREDUCE, x, y, n, L.FP32, 4, n * 4, 4)) / 4
        assert comm.sync() == 0
        print("single-rank allreduce 64 MiB: %.1f us, %.0f GB/s read+write" % (ms * 1e3, 2 * n * 4 / ms / 1e6))
        comm.destroy()
    elif case in ("allreduce", "ll"):
        cfg = L.CommConfig.default()
        cfg.hcclBufferSize = 128
        comm = H.Communicator.init_local(2, device=True, device_id=0, config=cfg)
        n = (16 << 20) if case == "allreduce" else (64 << 10)
        xs = [torch.rand(n, device="cuda") for _ in range(2)]
        ys = [torch.empty(n, device="cuda") for _ in range(2)]
        algo = L.ALGO_MESH if case == "allreduce" else L.ALGO_LL
        ms = _timed(lambda: comm.all_reduce(xs, ys, algo=algo))
        assert comm.sync() == 0, comm.describe_status()
        print("%s two virtual ranks, %d bytes: %.1f us" % (case, n * 4, ms * 1e3))
        comm.destroy()
    elif case == "moe":
        comm = H.Communicator.init_root(1, H.Communicator.get_root_info(), 0, device=True)
        T, Hd, E, k = 2048, 7168, 32, 8
        ex = moe.MoEExchange(comm, T, Hd, E, k, capacity_factor=1.1)
        x = torch.randn(T, Hd, device="cuda").to(torch.bfloat16)
        idx, gates = moe.route(T, E, k, 7, 0)
        out = torch.empty_like(x)

        def step():
            ex.dispatch(x, idx)
            ex.combine(gates, source="recv", out=out)
        ms = _timed(step)
        assert comm.sync() == 0
        print("moe dispatch+combine %d tokens: %.3f ms (%.0f MB each way)" % (T, ms, T * k * Hd * 2 / 1e6))
        ex.close()
        comm.destroy()
    else:
        raise SystemExit("unknown case " + case)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gemm")
