"""Side benchmarks reported inside bench.py's JSON line: the fused tensor-parallel MLP kernels (Llama-3-70B shapes:
8192 tokens, hidden 8192, FFN 28672 split over the ranks) next to cuBLAS + NCCL, and the MoE dispatch/combine exchange
next to NCCL all-to-all.  Device-timed with CUDA events, max over ranks."""
import json
import os

import torch

from . import fused_tp

TOKENS, HIDDEN, FFN = 8192, 8192, 28672


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops_sustained", 1387.8)), "measured"
    except Exception:
        return 1400.0, "fallback"


def _time(fn, iters, sync):
    for _ in range(3):
        fn()
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / iters
    sync()
    return ms


def other_collectives(comm, world, rank, dist, max_over_ranks, sync):
    """AllGather / ReduceScatter / Broadcast and AllReduce in bf16 and with max, 64 MiB per rank, next to NCCL
    (torch.distributed on the same stream).  Ours is issued by the C loop; both are device-timed, max over ranks."""
    from .. import _lib as L
    rows = {}
    mib = 64
    iters = 8

    def t_ours(coll, send, recv, count, dtype, **kw):
        comm.repeat(coll, send, recv, count, dtype, 3, **kw)
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        comm.repeat(coll, send, recv, count, dtype, iters, **kw)
        b.record()
        torch.cuda.synchronize()
        assert comm.sync() == 0, comm.describe_status()
        return max_over_ranks(a.elapsed_time(b) / iters)

    def t_nccl(fn):
        return max_over_ranks(_time(fn, iters, sync))

    def row(name, ours_ms, nccl_ms, nbytes):
        rows[name] = {"bytes_per_rank": nbytes, "ours_us": round(ours_ms * 1e3, 1), "nccl_us": round(nccl_ms * 1e3, 1),
                      "ours_GBps": round(nbytes / ours_ms / 1e6, 1), "nccl_GBps": round(nbytes / nccl_ms / 1e6, 1),
                      "speedup_vs_nccl": round(nccl_ms / ours_ms, 3)}

    for dt, hd, name in ((torch.bfloat16, L.BFP16, "bf16"), (torch.float32, L.FP32, "fp32")):
        es = 2 if dt == torch.bfloat16 else 4
        n = (mib << 20) // es
        small = torch.randn(n, device="cuda").to(dt)
        big = torch.randn(n * world, device="cuda").to(dt)
        big2 = torch.empty_like(big)
        small2 = torch.empty_like(small)
        # AllGather: 64 MiB sent by each rank; bandwidth counted on the gathered bytes per rank as hccl_test does for the send size
        row("allgather_%s" % name, t_ours(L.ALLGATHER, small, big2, n, hd), t_nccl(lambda: dist.all_gather_into_tensor(big2, small)), n * es)
        row("reducescatter_sum_%s" % name, t_ours(L.REDUCE_SCATTER, big, small2, n, hd), t_nccl(lambda: dist.reduce_scatter_tensor(small2, big)), n * es)
        if name == "bf16":
            row("allreduce_sum_bf16", t_ours(L.ALLREDUCE, small, small2, n, hd), t_nccl(lambda: dist.all_reduce(small2)), n * es)
        else:
            row("allreduce_max_fp32", t_ours(L.ALLREDUCE, small, small2, n, hd, op=L.MAX),
                t_nccl(lambda: dist.all_reduce(small2, op=dist.ReduceOp.MAX)), n * es)
            row("broadcast_fp32", t_ours(L.BROADCAST, small, small, n, hd, root=0), t_nccl(lambda: dist.broadcast(small2, src=0)), n * es)
        del small, big, big2, small2
    return rows


def run(comm, world, rank, dist, max_over_ranks, sync, time_steps):
    out = {}
    peak_tflops, peak_kind = _peaks()
    link_gbs = 770.0
    fl = FFN // world
    ms_rows = TOKENS // world
    g = torch.Generator(device="cuda").manual_seed(0)
    x_shard = torch.randn(ms_rows, HIDDEN, device="cuda", generator=g).to(torch.bfloat16)
    w_up = (torch.randn(fl, HIDDEN, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    w_down = (torch.randn(HIDDEN, fl, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    h = torch.randn(TOKENS, fl, device="cuda", generator=g).to(torch.bfloat16)
    y = torch.empty(TOKENS, fl, device="cuda", dtype=torch.bfloat16)
    o = torch.empty(ms_rows, HIDDEN, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * TOKENS * HIDDEN * fl
    comm_bytes = (world - 1) / world * TOKENS * HIDDEN * 2
    roof_ms = max(flops / (peak_tflops * 1e9), comm_bytes / (link_gbs * 1e6))
    iters = 10
    # ---- all-gather(X) -> X W_up^T
    t = max_over_ranks(_time(lambda: fused_tp.all_gather_matmul(comm, x_shard, w_up, out=y), iters, sync))
    assert comm.sync() == 0, comm.describe_status()
    row = {"ms": round(t, 4), "tflops_per_gpu": round(flops / t / 1e9, 1), "roofline_ms": round(roof_ms, 4),
           "roofline_fraction": round(roof_ms / t, 3), "roofline_kind": "of %s peak (%.0f TFLOP/s sustained, %.0f GB/s link)" % (peak_kind, peak_tflops, link_gbs)}
    xfull = torch.empty(TOKENS, HIDDEN, device="cuda", dtype=torch.bfloat16)
    if dist is not None:
        def base_ag():
            dist.all_gather_into_tensor(xfull, x_shard)
            torch.matmul(xfull, w_up.t(), out=y)
    else:
        def base_ag():
            torch.matmul(x_shard, w_up.t(), out=y)
    tb = max_over_ranks(_time(base_ag, iters, sync))
    row["cublas_nccl_ms"] = round(tb, 4)
    row["speedup_vs_cublas_nccl"] = round(tb / t, 3)
    # numerics of the fused kernel against the cuBLAS + NCCL result of the same operands (both bf16 outputs)
    y_ref = y.clone()
    fused_tp.all_gather_matmul(comm, x_shard, w_up, out=y)
    assert comm.sync() == 0, comm.describe_status()
    err = float((y.float() - y_ref.float()).norm() / (y_ref.float().norm() + 1e-12))
    row["rel_err_vs_cublas_nccl"] = round(max_over_ranks(err), 6)
    if world > 1:
        # the same with the shard in registered symmetric memory: the peers pull it in place, no staging copy
        handle, bufs = comm.symmetric_empty(x_shard.numel(), torch.bfloat16)
        xz = bufs[0].view_as(x_shard)
        xz.copy_(x_shard)
        tz = max_over_ranks(_time(lambda: fused_tp.all_gather_matmul(comm, xz, w_up, out=y), iters, sync))
        assert comm.sync() == 0, comm.describe_status()
        row["registered_shard_ms"] = round(tz, 4)
        row["registered_shard_speedup_vs_cublas_nccl"] = round(tb / tz, 3)
        row["registered_shard_roofline_fraction"] = round(roof_ms / tz, 3)
        err = float((y.float() - y_ref.float()).norm() / (y_ref.float().norm() + 1e-12))
        row["registered_shard_rel_err"] = round(max_over_ranks(err), 6)
        del xz, bufs
        comm.mem_free(handle)
    del y_ref
    out["ag_gemm"] = row
    # ---- H W_down^T -> reduce-scatter
    t = max_over_ranks(_time(lambda: fused_tp.matmul_reduce_scatter(comm, h, w_down, out=o), iters, sync))
    assert comm.sync() == 0, comm.describe_status()
    row = {"ms": round(t, 4), "tflops_per_gpu": round(flops / t / 1e9, 1), "roofline_ms": round(roof_ms, 4), "roofline_fraction": round(roof_ms / t, 3)}
    part = torch.empty(TOKENS, HIDDEN, device="cuda", dtype=torch.bfloat16)
    if dist is not None:
        def base_rs():
            torch.matmul(h, w_down.t(), out=part)
            dist.reduce_scatter_tensor(o, part)
    else:
        def base_rs():
            torch.matmul(h, w_down.t(), out=part)
    tb = max_over_ranks(_time(base_rs, iters, sync))
    row["cublas_nccl_ms"] = round(tb, 4)
    row["speedup_vs_cublas_nccl"] = round(tb / t, 3)
    o_ref = o.clone()
    fused_tp.matmul_reduce_scatter(comm, h, w_down, out=o)
    assert comm.sync() == 0, comm.describe_status()
    err = float((o.float() - o_ref.float()).norm() / (o_ref.float().norm() + 1e-12))
    row["rel_err_vs_cublas_nccl"] = round(max_over_ranks(err), 6)
    del o_ref
    out["gemm_rs"] = row
    out["shape"] = {"tokens": TOKENS, "hidden": HIDDEN, "ffn_per_gpu": fl, "dtype": "bf16"}
    del x_shard, w_up, w_down, h, y, o, xfull, part
    if dist is not None:
        try:
            out["collectives_vs_nccl"] = other_collectives(comm, world, rank, dist, max_over_ranks, sync)
        except Exception as e:  # a side table never takes the rest down
            out["collectives_vs_nccl"] = {"error": repr(e)[:300]}
    try:
        from . import moe
        out["moe"] = moe.bench(comm, world, rank, dist, max_over_ranks, sync)
    except ImportError:
        pass
    return out
