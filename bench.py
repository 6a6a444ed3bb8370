#!/usr/bin/env python
"""Headline benchmark: hccl_test-shaped AllReduce (sum, fp32) on N B200 GPUs, next to NCCL on the same box.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 20 --warmup 5

A "step" is one HcclAllReduce of the headline message (64 MiB per rank, fp32, sum, algorithm chosen by the
selector).  The K timed steps are issued back to back from C (the way the C program hccl_test does), bracketed by a
barrier + torch.cuda.synchronize() and timed with CUDA events on the launching stream; the reported time is the max
over ranks.  The NCCL baseline is ncclAllReduce issued by the same kind of loop on the same buffers.  Successive steps rotate through buffer sets whose total
size exceeds the 126 MB L2, so no step finds its input in cache.  The JSON line also carries a size sweep
(8 KiB .. 256 MiB: aveg_time us / alg_bandwidth GB/s for this library and for NCCL), the end-to-end number
(pinned host -> device copy of the input, the collective, device -> host copy of the result, every step), SM clock
samples taken during the timed region, and the count of this library's kernel launches in the timed region.

`--impl reference` reports that the Ascend reference cannot run here (it needs the CANN toolkit, Ascend NPUs and a
closed platform library; it has no Python package to install).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

HEADLINE_BYTES = 64 << 20
METRIC = "allreduce_alg_bandwidth_GBps_64MiB_fp32_sum"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.rows = []
        self._stop = threading.Event()
        self._th = None

    def _run(self):
        q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        self._th = threading.Thread(target=self._run, daemon=True)
        self._th.start()

    def stop(self):
        self._stop.set()
        if self._th:
            self._th.join(timeout=6)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for i, n in enumerate(names):
                    if r[3 + i].lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def time_steps(fn, steps, warmup, sync):
    """Device time of `steps` calls of fn(i) in ms (CUDA events on the current stream), after `warmup` untimed calls."""
    import torch
    for i in range(warmup):
        fn(i)
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    sync()
    return ms


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep-max", type=int, default=256 << 20, help="largest per-rank message of the size sweep (bytes)")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the fused-TP / MoE / AllGather side benchmarks")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "yzh1703456/cann-hccl needs the CANN toolkit, Ascend NPUs and the closed "
                          "libhccl_plf.so; the tree has no setup.py/pyproject.toml, so pip cannot install it"}))
        return 0

    import torch
    import torch.distributed as dist
    import cann_hccl_b200 as H
    from cann_hccl_b200 import _lib as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1 and args.gpus == 1, "launch with torchrun --nproc-per-node == --gpus"
    torch.cuda.set_device(local_rank)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    # staging of 640 MB per direction (HCCL_BUFFSIZE semantics; the default is 200): every message of the sweep and the
    # 8 x 64 MiB AllGather / ReduceScatter of the side table then run as one launch instead of a staging loop
    cfg = L.CommConfig.default()
    cfg.hcclBufferSize = int(os.environ.get("HCCL_BUFFSIZE", "640"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        blob = [H.Communicator.get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(blob, src=0)
        comm = H.Communicator.init_root(world, blob[0], rank, config=cfg, device=True)
    else:
        comm = H.Communicator.init_root(1, H.Communicator.get_root_info(), 0, config=cfg, device=True)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if world > 1:
        try:
            comm.calibrate()
        except H.HcclError as e:  # calibration is an optimisation; the default model still selects sensibly
            if rank == 0:
                print("calibration skipped: %s" % e, file=sys.stderr)

    # ---------------------------------------------------------------- headline: 64 MiB fp32 sum, auto-selected algorithm
    n = HEADLINE_BYTES // 4
    nset = 4  # 4 x (64 MiB in + 64 MiB out) = 512 MiB rotated > 126 MB L2
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)

    # the nset buffer sets are contiguous slices of one allocation so that the C-level loop can rotate through them
    big_in = torch.empty(n * nset, device="cuda")
    big_out = torch.empty(n * nset, device="cuda")
    big_in.uniform_(-1, 1, generator=g)
    ins = [big_in[i * n:(i + 1) * n] for i in range(nset)]
    outs = [big_out[i * n:(i + 1) * n] for i in range(nset)]

    def step(i):
        comm.all_reduce(ins[i % nset], outs[i % nset])

    def run_steps(k):
        # hccl_test style: k back-to-back HcclAllReduce calls issued from C, buffer set i % nset for call i
        comm.repeat(L.ALLREDUCE, big_in, big_out, n, L.FP32, k, HEADLINE_BYTES, nset)

    def timed(fn_k, k):
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn_k(k)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        sync()
        return ms

    # correctness first (check_result): against NCCL when there are peers, against the input itself otherwise
    step(0)
    assert comm.sync() == 0, comm.describe_status()
    if world > 1:
        ref = ins[0].clone()
        dist.all_reduce(ref)
        check = bool(torch.allclose(outs[0], ref, rtol=1e-5, atol=1e-5))
    else:
        check = bool(torch.equal(outs[0], ins[0]))
    sampler = ClockSampler(local_rank)
    sync()
    sampler.start()
    run_steps(warmup)            # untimed warm-up steps
    sync()
    launches0 = comm.stats()["launches"]
    ms = timed(run_steps, steps)
    launches = comm.stats()["launches"] - launches0
    clocks = sampler.stop()
    assert comm.sync() == 0, comm.describe_status()
    ms = max_over_ranks(ms)
    ms_per_step = ms / steps
    value = HEADLINE_BYTES / (ms_per_step * 1e-3) / 1e9
    algo = comm.select(L.ALLREDUCE, n, L.FP32)[0]

    nccl_ms = None
    if world > 1:
        def nccl_steps(k):
            # the baseline issued the same way: ncclAllReduce in a C loop on the same rotating buffers (in place)
            rc = comm.nccl_allreduce_repeat(big_out, big_out, n, L.FP32, k, HEADLINE_BYTES, nset)
            assert rc == 0, "NCCL baseline unavailable (%d)" % rc
        nccl_steps(warmup)
        nccl_ms = max_over_ranks(timed(nccl_steps, steps)) / steps

    # ---------------------------------------------------------------- end to end through the public API, host to host
    hin = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)]
    hout = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)]
    for h in hin:
        h.uniform_(-1, 1)
    e2e_steps = max(3, min(steps, 10))

    def e2e_step(i):
        d_in, d_out = ins[i % nset], outs[i % nset]
        d_in.copy_(hin[i % 2], non_blocking=True)        # H2D of this step's input (pinned)
        comm.all_reduce(d_in, d_out)
        hout[i % 2].copy_(d_out, non_blocking=True)       # D2H of this step's result

    e2e_ms = max_over_ranks(time_steps(e2e_step, e2e_steps, 3, sync)) / e2e_steps
    assert comm.sync() == 0, comm.describe_status()
    e2e_value = HEADLINE_BYTES / (e2e_ms * 1e-3) / 1e9

    # ---------------------------------------------------------------- hccl_test-shaped size sweep
    sweep = []
    if not args.no_sweep:
        size = 8 << 10
        sw_in = torch.empty(max(args.sweep_max, HEADLINE_BYTES) // 4, device="cuda")
        sw_in.uniform_(-1, 1)
        sw_out = torch.empty_like(sw_in)
        zc_buf = zc_handle = None
        if world > 1 and comm.has_nvls():
            zc_handle, (zc_buf,) = comm.symmetric_empty(sw_in.numel(), torch.float32)
            zc_buf.uniform_(-1, 1)
        while size <= args.sweep_max:
            cnt = size // 4
            # rotate through disjoint windows of the big buffers so that small messages also miss L2 between iterations
            nwin = max(1, min(16, sw_in.numel() // cnt))
            iters = 50 if size <= (1 << 20) else (20 if size <= (32 << 20) else 8)

            def ours(k, cnt=cnt, nwin=nwin, size=size):
                comm.repeat(L.ALLREDUCE, sw_in, sw_out, cnt, L.FP32, k, size, nwin)
            ours(5)
            t_ours = max_over_ranks(timed(ours, iters)) / iters
            row = {"data_size": size, "aveg_time_us": round(t_ours * 1e3, 2), "alg_bandwidth_GBps": round(size / t_ours / 1e6, 2),
                   "algo": comm.select(L.ALLREDUCE, cnt, L.FP32)[0]}
            if world > 1:
                def nccl(k, cnt=cnt, nwin=nwin, size=size):
                    rc = comm.nccl_allreduce_repeat(sw_out, sw_out, cnt, L.FP32, k, size, nwin)
                    assert rc == 0
                nccl(5)
                t_n = max_over_ranks(timed(nccl, iters)) / iters
                row["nccl_time_us"] = round(t_n * 1e3, 2)
                row["nccl_alg_bandwidth_GBps"] = round(size / t_n / 1e6, 2)
            if world > 1 and zc_buf is not None and size >= (1 << 20):
                # same collective on buffers in registered symmetric memory: the zero-copy NVLS path (in place)
                def zc(k, cnt=cnt, nwin=nwin, size=size):
                    comm.repeat(L.ALLREDUCE, zc_buf, zc_buf, cnt, L.FP32, k, size, nwin)
                zc(max(5, nwin))
                t_z = max_over_ranks(timed(zc, iters)) / iters
                row["zero_copy_time_us"] = round(t_z * 1e3, 2)
                row["zero_copy_alg_bandwidth_GBps"] = round(size / t_z / 1e6, 2)
            sweep.append(row)
            size *= 2
        assert comm.sync() == 0, comm.describe_status()
        del sw_in, sw_out
        if zc_handle is not None:
            del zc_buf
            comm.mem_free(zc_handle)

    extras = {}
    if not args.no_extras:
        try:
            from cann_hccl_b200.parallel import bench_extras
            extras = bench_extras.run(comm, world, rank, dist if world > 1 else None, max_over_ranks, sync, time_steps)
        except ImportError:
            extras = {}
        except Exception as e:  # side benchmarks never take the headline down
            extras = {"error": repr(e)[:300]}

    result = {
        "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic (uniform[-1,1) seeded 1234+rank)",
        "config": {"model": "hccl_test all_reduce_test -d fp32 -o sum", "global_batch": world, "seq_len": n,
                   "message_bytes_per_rank": HEADLINE_BYTES, "parallelism": "allreduce%d" % world, "algorithm": algo,
                   "nvls": comm.has_nvls(), "l2_policy": "4 rotating buffer sets, 512 MiB total > 126 MB L2", "staging_mb": int(cfg.hcclBufferSize)},
        "check_result": "success" if check else "failed",
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 3), "unit": "GB/s", "h2d_bytes_per_step": HEADLINE_BYTES, "d2h_bytes_per_step": HEADLINE_BYTES,
                "ms_per_step": round(e2e_ms, 5)},
        "gpu_launches": int(launches),
        "nccl": None if nccl_ms is None else {"ms_per_step": round(nccl_ms, 5), "alg_bandwidth_GBps": round(HEADLINE_BYTES / nccl_ms / 1e6, 3)},
        "vs_nccl": None if nccl_ms is None else round(nccl_ms / ms_per_step, 4),
        "sweep": sweep,
        "extras": extras,
        "cost_model": comm.stats()["model"],
    }
    comm.destroy()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))
    return 0 if check else 1


if __name__ == "__main__":
    sys.exit(main())
