"""Side tables of bench.py's JSON line: the sweeps of the other collectives next to NCCL (AllGather, ReduceScatter,
Broadcast, Reduce, Scatter, Gather; recursive halving-doubling against ring), the fused tensor-parallel MLP kernels
(Llama-3-70B shapes: 8192 tokens, hidden 8192, FFN 28672 split over the ranks) next to cuBLAS + NCCL, and the MoE
dispatch / combine exchange next to NCCL all-to-all.  Everything is device-timed with CUDA events, max over ranks, and
every correctness figure printed here is also checked: a result out of tolerance is listed in `failures`, which makes
bench.py exit non-zero."""
import json
import os

import torch

from cann_hccl_b200 import _lib as L
from cann_hccl_b200.parallel import fused_tp

TOKENS, HIDDEN, FFN = 8192, 8192, 28672
HERE = os.path.dirname(os.path.abspath(__file__))


def peaks():
    """Measured peaks of this pool (written by the driver next to this file); the stated fallback when the file is absent."""
    try:
        with open(os.path.join(HERE, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]), "kind": "measured"}
    except Exception:
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "kind": "fallback"}


def _time(fn, iters, sync, warm=3):
    for _ in range(warm):
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


def collective_sweeps(comm, world, rank, dist, max_over_ranks, sync, max_bytes, failures):
    """AllGather / ReduceScatter (sum; fp32 and bf16) and Broadcast / Reduce / Scatter / Gather (root 0, fp32) from 1 KiB
    to `max_bytes` per rank in steps of 4x, this library (auto-selected; ring and halving-doubling forced where both exist)
    next to NCCL through torch.distributed on the same stream.  Sizes are bytes of the collective's count argument."""
    out = {}
    sizes = []
    s = 1 << 10
    while s <= max_bytes:
        sizes.append(s)
        s *= 4
    if sizes[-1] != max_bytes:
        sizes.append(max_bytes)

    def t_ours(coll, send, recv, count, dtype, iters, **kw):
        comm.repeat(coll, send, recv, count, dtype, 2, **kw)
        best = None
        for _ in range(2):  # the better of two timed loops: one stall of a shared host does not decide a row
            sync()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            comm.repeat(coll, send, recv, count, dtype, iters, **kw)
            b.record()
            torch.cuda.synchronize()
            assert comm.sync() == 0, comm.describe_status()
            t = max_over_ranks(a.elapsed_time(b) / iters)
            best = t if best is None else min(best, t)
        return best

    specs = [("allgather", L.ALLGATHER, (torch.float32, torch.bfloat16), (L.ALGO_RING, L.ALGO_RHD)),
             ("reducescatter", L.REDUCE_SCATTER, (torch.float32, torch.bfloat16), (L.ALGO_RING, L.ALGO_RHD)),
             ("broadcast", L.BROADCAST, (torch.float32,), ()), ("reduce", L.REDUCE, (torch.float32,), (L.ALGO_MESH_PIPE, L.ALGO_TREE)),
             ("scatter", L.SCATTER, (torch.float32,), ()), ("gather", L.GATHER, (torch.float32,), ())]
    hd = {torch.float32: L.FP32, torch.bfloat16: L.BFP16}
    for name, coll, dtypes, forced in specs:
        for dt in dtypes:
            es = dt.itemsize
            rows = []
            big_in = coll in (L.REDUCE_SCATTER, L.SCATTER)
            big_out = coll in (L.ALLGATHER, L.GATHER)
            nmax = sizes[-1] // es
            g = torch.Generator(device="cuda").manual_seed(4321 + rank)
            src = torch.randn(nmax * (world if big_in else 1), device="cuda", generator=g).to(dt)
            dst = torch.empty(nmax * (world if big_out else 1), device="cuda", dtype=dt)
            for size in sizes:
                n = size // es
                iters = 20 if size <= (1 << 20) else (8 if size <= (64 << 20) else 3)
                send = src[:n * (world if big_in else 1)]
                recv = dst[:n * (world if big_out else 1)]
                if coll == L.BROADCAST:
                    recv = send
                row = {"data_size": size}
                t = t_ours(coll, send, recv, n, hd[dt], iters, root=0)
                row["aveg_time_us"] = round(t * 1e3, 2)
                row["alg_bandwidth_GBps"] = round(size / t / 1e6, 2)
                row["algo"] = comm.trace()[-1]["algo"]
                for fa in forced:
                    if size >= (64 << 10) and (world & (world - 1)) == 0:
                        tf = t_ours(coll, send, recv, n, hd[dt], iters, root=0, algo=fa)
                        row[L.ALGO_NAMES[fa] + "_us"] = round(tf * 1e3, 2)
                if dist is not None:
                    fn = {L.ALLGATHER: lambda: dist.all_gather_into_tensor(recv, send),
                          L.REDUCE_SCATTER: lambda: dist.reduce_scatter_tensor(recv, send),
                          L.BROADCAST: lambda: dist.broadcast(send, src=0),
                          L.REDUCE: lambda: dist.reduce(send, dst=0),
                          L.SCATTER: lambda: dist.scatter(recv, list(send.chunk(world)) if rank == 0 else None, src=0),
                          L.GATHER: lambda: dist.gather(send, list(recv.chunk(world)) if rank == 0 else None, dst=0)}[coll]
                    tn = min(max_over_ranks(_time(fn, iters, sync, warm=2)), max_over_ranks(_time(fn, iters, sync, warm=0)))
                    row["nccl_time_us"] = round(tn * 1e3, 2)
                    row["nccl_alg_bandwidth_GBps"] = round(size / tn / 1e6, 2)
                    row["vs_nccl"] = round(tn / t, 3)
                rows.append(row)
            # check_result at one mid size against NCCL's result of the same inputs
            if dist is not None:
                n = min(nmax, (4 << 20) // es)
                send = src[:n * (world if big_in else 1)].clone()
                ours_out = torch.zeros(n * (world if big_out else 1), device="cuda", dtype=dt)
                ref_out = torch.zeros_like(ours_out)
                if coll == L.ALLGATHER:
                    comm.all_gather(send, ours_out); dist.all_gather_into_tensor(ref_out, send)
                elif coll == L.REDUCE_SCATTER:
                    comm.reduce_scatter(send, ours_out); dist.reduce_scatter_tensor(ref_out, send)
                elif coll == L.BROADCAST:
                    ours_out = send.clone(); ref_out = send.clone()
                    comm.broadcast(ours_out, 0); dist.broadcast(ref_out, src=0)
                elif coll == L.REDUCE:
                    comm.reduce(send, ours_out, 0); ref_out = send.clone(); dist.reduce(ref_out, dst=0)
                elif coll == L.SCATTER:
                    comm.scatter(send, ours_out, 0); dist.scatter(ref_out, list(send.chunk(world)) if rank == 0 else None, src=0)
                else:
                    comm.gather(send, ours_out, 0); dist.gather(send, list(ref_out.chunk(world)) if rank == 0 else None, dst=0)
                assert comm.sync() == 0, comm.describe_status()
                torch.cuda.synchronize()
                rooted_result_elsewhere = coll in (L.REDUCE, L.GATHER) and rank != 0
                tol = 1e-5 * world if dt == torch.float32 else 2e-2 * world
                okay = rooted_result_elsewhere or bool(torch.allclose(ours_out.float(), ref_out.float(), rtol=tol, atol=tol))
                ok_all = max_over_ranks(0.0 if okay else 1.0) == 0.0
                if not ok_all:
                    failures.append("%s_%s check_result" % (name, "fp32" if dt == torch.float32 else "bf16"))
            out["%s_%s" % (name, "fp32" if dt == torch.float32 else "bf16")] = {"check_result": "n/a" if dist is None else ("success" if ok_all else "failed"),
                                                                                 "rows": rows}
            del src, dst
    return out


def fused_tp_rows(comm, world, rank, dist, max_over_ranks, sync, failures):
    out = {}
    pk = peaks()
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
    # a kernel timed in isolation runs at burst clocks: its roofline is the measured burst cuBLAS rate, and the measured
    # peer-copy rate for what must cross NVLink
    roof_ms = max(flops / (pk["bf16_tflops"] * 1e9), comm_bytes / (link_gbs * 1e6))
    kind = "of %s (%.0f TFLOP/s cuBLAS bf16 burst, %.0f GB/s peer copy)" % (pk["kind"], pk["bf16_tflops"], link_gbs)
    iters = 10

    def rel(a, b):
        return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))

    # ---- all-gather(X) -> X W_up^T
    t = max_over_ranks(_time(lambda: fused_tp.all_gather_matmul(comm, x_shard, w_up, out=y), iters, sync))
    assert comm.sync() == 0, comm.describe_status()
    row = {"ms": round(t, 4), "tflops_per_gpu": round(flops / t / 1e9, 1), "roofline_ms": round(roof_ms, 4),
           "roofline_fraction": round(roof_ms / t, 3), "roofline_kind": kind}
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
    y_ref = y.clone()
    fused_tp.all_gather_matmul(comm, x_shard, w_up, out=y)
    assert comm.sync() == 0, comm.describe_status()
    row["rel_err_vs_cublas_nccl"] = round(max_over_ranks(rel(y, y_ref)), 6)
    if row["rel_err_vs_cublas_nccl"] > 1e-2:
        failures.append("ag_gemm rel_err")
    if world > 1:
        handle, bufs = comm.symmetric_empty(x_shard.numel(), torch.bfloat16)
        xz = bufs[0].view_as(x_shard)
        xz.copy_(x_shard)
        tz = max_over_ranks(_time(lambda: fused_tp.all_gather_matmul(comm, xz, w_up, out=y), iters, sync))
        assert comm.sync() == 0, comm.describe_status()
        row["registered_shard_ms"] = round(tz, 4)
        row["registered_shard_speedup_vs_cublas_nccl"] = round(tb / tz, 3)
        row["registered_shard_roofline_fraction"] = round(roof_ms / tz, 3)
        row["registered_shard_rel_err"] = round(max_over_ranks(rel(y, y_ref)), 6)
        if row["registered_shard_rel_err"] > 1e-2:
            failures.append("ag_gemm registered rel_err")
        del xz, bufs
        comm.mem_free(handle)
    del y_ref
    out["ag_gemm"] = row
    # ---- H W_down^T -> reduce-scatter
    t = max_over_ranks(_time(lambda: fused_tp.matmul_reduce_scatter(comm, h, w_down, out=o), iters, sync))
    assert comm.sync() == 0, comm.describe_status()
    row = {"ms": round(t, 4), "tflops_per_gpu": round(flops / t / 1e9, 1), "roofline_ms": round(roof_ms, 4), "roofline_fraction": round(roof_ms / t, 3),
           "roofline_kind": kind}
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
    o_ref = (o if dist is not None else part).clone()
    fused_tp.matmul_reduce_scatter(comm, h, w_down, out=o)
    assert comm.sync() == 0, comm.describe_status()
    row["rel_err_vs_cublas_nccl"] = round(max_over_ranks(rel(o, o_ref)), 6)
    if row["rel_err_vs_cublas_nccl"] > 2e-2:
        failures.append("gemm_rs rel_err")
    out["gemm_rs"] = row
    out["shape"] = {"tokens": TOKENS, "hidden": HIDDEN, "ffn_per_gpu": fl, "dtype": "bf16"}
    return out


def run(comm, world, rank, dist, max_over_ranks, sync, max_bytes, failures, want=("collectives", "fused_tp", "moe")):
    out = {}
    if "fused_tp" in want:
        try:
            out.update(fused_tp_rows(comm, world, rank, dist, max_over_ranks, sync, failures))
        except Exception as e:  # a side table never takes the headline down, but it is on record as a failure
            out["fused_tp_error"] = repr(e)[:300]
            failures.append("fused_tp raised")
        torch.cuda.empty_cache()
    if "collectives" in want and dist is not None:
        try:
            out["collective_sweeps"] = collective_sweeps(comm, world, rank, dist, max_over_ranks, sync, max_bytes, failures)
        except Exception as e:
            out["collective_sweeps"] = {"error": repr(e)[:300]}
            failures.append("collective sweeps raised")
        torch.cuda.empty_cache()
    if "moe" in want:
        try:
            from cann_hccl_b200.parallel import moe
            out["moe"] = moe.bench(comm, world, rank, dist, max_over_ranks, sync)
            if out["moe"].get("check_max_abs_err", 0) > 0.25:
                failures.append("moe check_max_abs_err")
            if out["moe"].get("alltoallv_api_check_max_abs_err", 0) > 0.25:
                failures.append("moe alltoallv_api_check_max_abs_err")
        except Exception as e:
            out["moe"] = {"error": repr(e)[:300]}
            failures.append("moe raised")
    return out
