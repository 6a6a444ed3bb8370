#!/usr/bin/env python
"""Headline benchmark: hccl_test-shaped AllReduce (sum, fp32) on N B200 GPUs, next to NCCL on the same box.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 20 --warmup 5

A "step" is one HcclAllReduce of the headline message (64 MiB per rank, fp32, sum, algorithm chosen by the selector,
whose tables the communicator measured when it was created).  The K timed steps are issued back to back from C (the
way the C program hccl_test does), bracketed by a barrier + torch.cuda.synchronize() and timed with CUDA events on the
launching stream; the time is the max over ranks.  The K-step block is repeated until at least 250 ms have been
timed, and the median block is reported (so that the clock samples cover a loaded GPU).  The NCCL baseline is
ncclAllReduce issued by the same kind of loop on the same buffers.  Successive steps rotate through buffer sets whose
total size exceeds the 126 MB L2, so no step finds its input in cache.  The JSON line also carries:
  sweep            AllReduce 8 KiB .. 1 GiB, sum fp32 with every algorithm forced next to `auto` and NCCL; from 1 MiB on also
                   both libraries on registered memory (this library's symmetric pool, NCCL's registered pool)
  sweep_variants   the same sizes for max / bf16 (auto and NCCL)
  extras           the other collectives' sweeps, the fused tensor-parallel kernels and the MoE exchange (bench_extras.py)
  e2e              pinned host -> device copy of the input, the collective, device -> host copy of the result, every step,
                   for this library and for NCCL
plus SM clock samples taken during the timed region and the count of this library's kernel launches in it.
Every correctness figure in the line is checked; a figure out of tolerance makes the exit code non-zero.

`--impl reference`: the Ascend reference cannot run here (it needs the CANN toolkit, Ascend NPUs and a closed platform
library, and has no Python package to install), which the line says in `unavailable`; the same line carries, under
`stand_in`, the baseline that the benchmark definition names for this box: NCCL AllReduce of the same config through
torch.distributed only (this library is not imported on that path).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

HEADLINE_BYTES = 64 << 20
METRIC = "allreduce_alg_bandwidth_GBps_64MiB_fp32_sum"
MIN_TIMED_MS = 1000.0
UNAVAILABLE = ("yzh1703456/cann-hccl needs the CANN toolkit, Ascend NPUs and the closed libhccl_plf.so; the tree has no "
               "setup.py/pyproject.toml, so pip cannot install it")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs.  Queries only: through the management
    library's Python binding (a sample takes well under a millisecond), or nvidia-smi when the binding is missing."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index):
        self.index = index
        self.sm, self.mx, self.reasons = [], [], set()
        self._stop = threading.Event()
        self._th = None
        self._nv = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].strip().isdigit() else index
            self._nv = (pynvml, pynvml.nvmlDeviceGetHandleByIndex(phys))
        except Exception:
            self._nv = None

    def _sample_nvml(self):
        nv, h = self._nv
        self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
        self.mx.append(float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)))
        bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
        for name, bit in self.REASONS:
            if bits & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q, "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip()
        r = [c.strip() for c in out.splitlines()[0].split(",")]
        self.sm.append(float(r[0]))
        self.mx.append(float(r[1]))
        for i, (name, _) in enumerate(self.REASONS):
            if r[2 + i].lower().startswith("active"):
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nv:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        self._th = threading.Thread(target=self._run, daemon=True)
        self._th.start()

    def stop(self):
        self._stop.set()
        if self._th:
            self._th.join(timeout=6)
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(self.mx) if self.mx else None, "reasons": sorted(self.reasons),
                "samples": len(sm), "source": "nvml" if self._nv else "nvidia-smi"}


def setup_dist(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1 and args.gpus == 1, "launch with torchrun --nproc-per-node == --gpus"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return torch, (dist if world > 1 else None), world, rank, local_rank


def timed_blocks(fn_k, steps, sync, max_over_ranks, est_ms=None):
    """Median over repeated K-step blocks (each bracketed by a barrier + synchronize on both sides); at least MIN_TIMED_MS in total."""
    import torch
    def block():
        sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn_k(steps)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        sync()
        return max_over_ranks(ms)
    first = block()
    nblocks = int(max(1, min(2000, MIN_TIMED_MS / max(first, 1e-3))))
    vals = sorted([first] + [block() for _ in range(nblocks)])
    return vals[len(vals) // 2], len(vals), sum(vals)


def e2e_rate(torch, step_fn, steps, sync, max_over_ranks):
    for i in range(3):
        step_fn(i)
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        step_fn(i)
    b.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(a.elapsed_time(b)) / steps
    sync()
    return ms


def reference_arm(args):
    """NCCL through torch.distributed only: the stand-in for the reference that cannot run on this hardware."""
    line = {"impl": "reference", "unavailable": UNAVAILABLE}
    try:
        torch, dist, world, rank, local_rank = setup_dist(args)
        warmup, steps = max(3, args.warmup), max(1, args.steps)
        n = HEADLINE_BYTES // 4
        nset = 4
        g = torch.Generator(device="cuda").manual_seed(1234 + rank)
        big = torch.empty(n * nset, device="cuda")
        big.uniform_(-1, 1, generator=g)
        bufs = [big[i * n:(i + 1) * n] for i in range(nset)]

        def sync():
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
                torch.cuda.synchronize()

        def mx(v):
            if dist is None:
                return v
            t = torch.tensor([v], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        def run_steps(k):
            for i in range(k):
                if dist is not None:
                    dist.all_reduce(bufs[i % nset])
                else:
                    bufs[(i + 1) % nset].copy_(bufs[i % nset])   # one rank: AllReduce is a copy
        sampler = ClockSampler(local_rank)
        sync()
        sampler.start()
        run_steps(warmup)
        ms, nblocks, total_ms = timed_blocks(run_steps, steps, sync, mx)
        clocks = sampler.stop()
        ms_per_step = ms / steps
        hin = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)]
        hout = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)]

        def e2e_step(i):
            d = bufs[i % nset]
            d.copy_(hin[i % 2], non_blocking=True)
            if dist is not None:
                dist.all_reduce(d)
            hout[i % 2].copy_(d, non_blocking=True)
        e2e_ms = e2e_rate(torch, e2e_step, max(3, min(steps, 10)), sync, mx)
        line["stand_in"] = {
            "impl": "nccl_baseline", "stands_in_for": "reference (unavailable: Ascend/CANN only)", "metric": METRIC,
            "value": round(HEADLINE_BYTES / (ms_per_step * 1e-3) / 1e9, 3), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": round(ms_per_step, 5), "blocks": nblocks, "timed_ms": round(total_ms, 1), "higher_is_better": True, "dtype": "fp32",
            "data": "synthetic (uniform[-1,1) seeded 1234+rank)", "clocks": clocks,
            "e2e": {"value": round(HEADLINE_BYTES / (e2e_ms * 1e-3) / 1e9, 3), "unit": "GB/s", "h2d_bytes_per_step": HEADLINE_BYTES,
                    "d2h_bytes_per_step": HEADLINE_BYTES, "ms_per_step": round(e2e_ms, 5)},
            "config": {"model": "ncclAllReduce via torch.distributed, fp32 sum, in place", "message_bytes_per_rank": HEADLINE_BYTES,
                       "l2_policy": "4 rotating buffers, 256 MiB total > 126 MB L2"}}
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
    except Exception as e:  # the line is printed whatever happens to the stand-in
        line["stand_in"] = {"impl": "nccl_baseline", "error": repr(e)[:300]}
        rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        emit_json(line)
    return 0


_REAL_STDOUT = None


def quiet_stdout():
    """Libraries print banners on the process's standard output (NCCL its version line, for one).  The result line has to be
    the only line there, so file descriptor 1 points at standard error until `emit_json` writes the result."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit_json(obj):
    sys.stdout.flush()
    if _REAL_STDOUT is not None:
        os.dup2(_REAL_STDOUT, 1)
    print(json.dumps(obj), flush=True)


def main():
    quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep-max", type=int, default=1 << 30, help="largest per-rank message of the sweeps (bytes)")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the other collectives / fused-TP / MoE side tables")
    ap.add_argument("--extras", default="collectives,fused_tp,moe", help="side tables to run: any of collectives, fused_tp, moe (comma-separated)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    # bounded device waits: a rank that is lost must not leave the other GPUs' CTAs polling for half an hour on a shared box
    os.environ.setdefault("HCCL_EXEC_TIMEOUT_MS", "30000")
    # a benchmark wants no quick verdict on a silent peer: on a loaded host a rank may be held up for seconds by allocations
    os.environ.setdefault("HCCL_HEARTBEAT_LOST_MS", "20000")
    torch, dist, world, rank, local_rank = setup_dist(args)
    import cann_hccl_b200 as H
    from cann_hccl_b200 import _lib as L
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    failures = []

    cfg = L.CommConfig.default()  # default staging (HCCL_BUFFSIZE semantics, 200 MB per direction) unless the environment says otherwise
    if world > 1:
        blob = [H.Communicator.get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(blob, src=0)
        comm = H.Communicator.init_root(world, blob[0], rank, config=cfg, device=True)
    else:
        comm = H.Communicator.init_root(1, H.Communicator.get_root_info(), 0, config=cfg, device=True)

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(flag):
        return max_over_ranks(0.0 if flag else 1.0) == 0.0

    # ---------------------------------------------------------------- headline: 64 MiB fp32 sum, auto-selected algorithm
    n = HEADLINE_BYTES // 4
    nset = 4  # 4 x (64 MiB in + 64 MiB out) = 512 MiB rotated > 126 MB L2
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    big_in = torch.empty(n * nset, device="cuda")
    big_out = torch.empty(n * nset, device="cuda")
    big_in.uniform_(-1, 1, generator=g)
    ins = [big_in[i * n:(i + 1) * n] for i in range(nset)]
    outs = [big_out[i * n:(i + 1) * n] for i in range(nset)]

    def run_steps(k):
        # hccl_test style: k back-to-back HcclAllReduce calls issued from C, buffer set i % nset for call i
        comm.repeat(L.ALLREDUCE, big_in, big_out, n, L.FP32, k, HEADLINE_BYTES, nset)

    comm.all_reduce(ins[0], outs[0])
    assert comm.sync() == 0, comm.describe_status()
    if dist is not None:
        ref = ins[0].clone()
        dist.all_reduce(ref)
        check = all_ok(bool(torch.allclose(outs[0], ref, rtol=1e-5, atol=1e-5)))
    else:
        check = bool(torch.equal(outs[0], ins[0]))
    if not check:
        failures.append("headline check_result")
    sampler = ClockSampler(local_rank)
    sync()
    sampler.start()
    run_steps(warmup)            # untimed warm-up steps
    sync()
    launches0 = comm.stats()["launches"]
    ms, nblocks, total_ms = timed_blocks(run_steps, steps, sync, max_over_ranks)
    launches = (comm.stats()["launches"] - launches0) // max(1, nblocks)
    clocks = sampler.stop()
    assert comm.sync() == 0, comm.describe_status()
    ms_per_step = ms / steps
    value = HEADLINE_BYTES / (ms_per_step * 1e-3) / 1e9
    algo = comm.select(L.ALLREDUCE, n, L.FP32)[0]

    nccl_ms = None
    if dist is not None:
        def nccl_steps(k):
            rc = comm.nccl_allreduce_repeat(big_out, big_out, n, L.FP32, k, HEADLINE_BYTES, nset)
            assert rc == 0, "NCCL baseline unavailable (%d)" % rc
        nccl_steps(warmup)
        nccl_ms = timed_blocks(nccl_steps, steps, sync, max_over_ranks)[0] / steps

    # ---------------------------------------------------------------- end to end through the public API, host to host
    hin = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)]
    hout = [torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(2)]
    for hbuf in hin:
        hbuf.uniform_(-1, 1)
    e2e_steps = max(3, min(steps, 10))

    def e2e_step(i):
        d_in, d_out = ins[i % nset], outs[i % nset]
        d_in.copy_(hin[i % 2], non_blocking=True)        # H2D of this step's input (pinned)
        comm.all_reduce(d_in, d_out)
        hout[i % 2].copy_(d_out, non_blocking=True)       # D2H of this step's result

    def e2e_step_nccl(i):
        d = outs[i % nset]
        d.copy_(hin[i % 2], non_blocking=True)
        dist.all_reduce(d)
        hout[i % 2].copy_(d, non_blocking=True)

    e2e_ms = e2e_rate(torch, e2e_step, e2e_steps, sync, max_over_ranks)
    assert comm.sync() == 0, comm.describe_status()
    e2e_nccl_ms = e2e_rate(torch, e2e_step_nccl, e2e_steps, sync, max_over_ranks) if dist is not None else None

    # ---------------------------------------------------------------- hccl_test-shaped AllReduce sweeps
    def sweep_rows(dtype_t, dtype_h, op_h, op_nccl, forced, registered=False):
        rows = []
        es = dtype_t.itemsize
        top = max(args.sweep_max, 8 << 10)
        # registered-memory columns: this library on tensors of its symmetric pool (ordinary torch tensors that the peers map:
        # zero-copy), and NCCL on tensors of its own registered pool (ncclMemAlloc + window registration through torch)
        z_in = z_out = nz = None
        if registered and comm.has_nvls():
            try:
                zpool = comm.symmetric_pool()
                with torch.cuda.use_mem_pool(zpool):
                    z_in = torch.empty(top // es, device="cuda", dtype=dtype_t)
                    z_out = torch.empty(top // es, device="cuda", dtype=dtype_t)
                z_in.uniform_(-1, 1)
            except Exception as e:
                z_in = z_out = None
                if rank == 0:
                    print("symmetric pool unavailable: %r" % (e,), file=sys.stderr)
            try:
                backend = dist.distributed_c10d._get_default_group()._get_backend(torch.device("cuda"))
                npool = torch.cuda.MemPool(backend.mem_allocator)
                with torch.cuda.use_mem_pool(npool):
                    nz = torch.empty(top // es, device="cuda", dtype=dtype_t)
                backend.register_mem_pool(npool)
                nz.uniform_(-1, 1)
            except Exception as e:
                nz = None
                if rank == 0:
                    print("NCCL registered pool unavailable: %r" % (e,), file=sys.stderr)
        cap_elems = min(2 * top, 2 << 30) // es               # up to 2 GiB per buffer: small messages rotate through windows
        sw_in = torch.empty(cap_elems, device="cuda", dtype=dtype_t)
        sw_in.uniform_(-1, 1)
        sw_out = torch.empty_like(sw_in)
        size = 8 << 10
        while size <= top:
            cnt = size // es
            nwin = max(1, min(16, sw_in.numel() // cnt))
            iters = 50 if size <= (1 << 20) else (20 if size <= (32 << 20) else (8 if size <= (256 << 20) else 4))

            def t_of(fn):
                fn(3)
                best = None
                for _ in range(2):  # the better of two timed loops: one stall of a shared host does not decide a row
                    sync()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    fn(iters)
                    b.record()
                    torch.cuda.synchronize()
                    t = max_over_ranks(a.elapsed_time(b) / iters)
                    best = t if best is None else min(best, t)
                sync()
                return best
            t_auto = t_of(lambda k: comm.repeat(L.ALLREDUCE, sw_in, sw_out, cnt, dtype_h, k, size, nwin, op=op_h))
            row = {"data_size": size, "aveg_time_us": round(t_auto * 1e3, 2), "alg_bandwidth_GBps": round(size / t_auto / 1e6, 2),
                   "algo": comm.select(L.ALLREDUCE, cnt, dtype_h, op_h)[0]}
            best_forced = None
            for an in forced:
                algo_id = L.ALGO_NAMES.index(an)
                if ("nvls" in an and not comm.has_nvls()) or (an == "ll" and size > (1 << 20)):
                    continue
                if an in ("mesh_oneshot", "nvls_oneshot") and size > (16 << 20) and world > 2:
                    continue   # every rank would pull (p-1) times the message
                if "pipe" in an and size < (1 << 20):
                    continue
                try:
                    tf = t_of(lambda k: comm.repeat(L.ALLREDUCE, sw_in, sw_out, cnt, dtype_h, k, size, nwin, op=op_h, algo=algo_id))
                except H.HcclError:
                    continue
                row[an + "_us"] = round(tf * 1e3, 2)
                best_forced = tf if best_forced is None else min(best_forced, tf)
            if best_forced is not None:
                row["auto_vs_best_forced"] = round(best_forced / t_auto, 3)
            if dist is not None:
                def nccl(k):
                    rc = comm.nccl_allreduce_repeat(sw_out, sw_out, cnt, dtype_h, k, size, nwin, op=op_h)
                    assert rc == 0
                t_n = t_of(nccl)
                row["nccl_time_us"] = round(t_n * 1e3, 2)
                row["nccl_alg_bandwidth_GBps"] = round(size / t_n / 1e6, 2)
                row["vs_nccl"] = round(t_n / t_auto, 3)
            if size >= (1 << 20):
                zwin = max(1, min(8, top // size))
                if z_in is not None:
                    t_z = t_of(lambda k: comm.repeat(L.ALLREDUCE, z_in, z_out, cnt, dtype_h, k, size, zwin, op=op_h))
                    row["registered_us"] = round(t_z * 1e3, 2)
                    row["registered_algo"] = comm.trace()[-1]["algo"]
                if nz is not None:
                    def nccl_reg(k):
                        for i in range(k):
                            o = (i % zwin) * cnt
                            dist.all_reduce(nz[o:o + cnt], op=op_nccl)
                    t_nz = t_of(nccl_reg)
                    row["nccl_registered_us"] = round(t_nz * 1e3, 2)
                    if z_in is not None:
                        row["registered_vs_nccl_registered"] = round(t_nz / t_z, 3)
            rows.append(row)
            size *= 2
        assert comm.sync() == 0, comm.describe_status()
        # check_result of this (type, operator) at 4 MiB against NCCL
        ok = True
        if dist is not None:
            cnt = (4 << 20) // es
            x = sw_in[:cnt].clone()
            y = torch.zeros_like(x)
            comm.all_reduce(x, y, op=op_h)
            assert comm.sync() == 0, comm.describe_status()
            refv = x.clone()
            dist.all_reduce(refv, op=op_nccl)
            tol = 1e-5 * world if dtype_t == torch.float32 else 2e-2 * world
            ok = all_ok(bool(torch.allclose(y.float(), refv.float(), rtol=tol, atol=tol)))
        if z_in is not None:
            # check_result of the zero-copy path at 4 MiB
            cnt = (4 << 20) // es
            x = z_in[:cnt].clone()
            refv = x.clone()
            dist.all_reduce(refv, op=op_nccl)
            z_in[:cnt].copy_(x)
            comm.all_reduce(z_in[:cnt], z_out[:cnt], op=op_h)
            assert comm.sync() == 0, comm.describe_status()
            tol = 1e-5 * world if dtype_t == torch.float32 else 2e-2 * world
            ok = ok and all_ok(bool(torch.allclose(z_out[:cnt].float(), refv.float(), rtol=tol, atol=tol)))
            del z_in, z_out, x, refv
            comm.release_symmetric_pool()
        del sw_in, sw_out, nz
        torch.cuda.empty_cache()
        return rows, ok

    sweep, variants = [], {}
    if not args.no_sweep and world > 1:
        forced = ["ll", "mesh_oneshot", "mesh", "ring", "rhd", "nvls_oneshot", "nvls", "mesh_pipe", "nvls_pipe"]
        sweep, ok = sweep_rows(torch.float32, L.FP32, L.SUM, dist.ReduceOp.SUM, forced, registered=True)
        if not ok:
            failures.append("sweep sum fp32 check_result")
        for name, dt, hd_, oph, opn in (("max_fp32", torch.float32, L.FP32, L.MAX, dist.ReduceOp.MAX),
                                        ("sum_bf16", torch.bfloat16, L.BFP16, L.SUM, dist.ReduceOp.SUM),
                                        ("max_bf16", torch.bfloat16, L.BFP16, L.MAX, dist.ReduceOp.MAX)):
            rows, ok = sweep_rows(dt, hd_, oph, opn, [])
            variants[name] = {"check_result": "success" if ok else "failed", "rows": rows}
            if not ok:
                failures.append("sweep %s check_result" % name)

    extras = {}
    if not args.no_extras:
        try:
            import bench_extras
            extras = bench_extras.run(comm, world, rank, dist, max_over_ranks, sync, min(args.sweep_max, 1 << 30), failures,
                                      want=tuple(x for x in args.extras.split(",") if x))
        except Exception as e:  # side tables never take the headline down, but the run is marked failed
            extras = {"error": repr(e)[:300]}
            failures.append("extras raised")

    st = comm.stats()
    result = {
        "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic (uniform[-1,1) seeded 1234+rank)",
        "config": {"model": "hccl_test all_reduce_test -d fp32 -o sum", "global_batch": world, "seq_len": n,
                   "message_bytes_per_rank": HEADLINE_BYTES, "parallelism": "allreduce%d" % world, "algorithm": algo,
                   "nvls": comm.has_nvls(), "l2_policy": "4 rotating buffer sets, 512 MiB total > 126 MB L2", "staging_mb": int(os.environ.get("HCCL_BUFFSIZE", "200")),
                   "timed_blocks": nblocks, "timed_ms": round(total_ms, 1), "exec_timeout_ms": int(os.environ["HCCL_EXEC_TIMEOUT_MS"])},
        "check_result": "success" if check else "failed",
        "failures": failures,
        "clocks": clocks,
        "e2e": {"value": round(HEADLINE_BYTES / (e2e_ms * 1e-3) / 1e9, 3), "unit": "GB/s", "h2d_bytes_per_step": HEADLINE_BYTES,
                "d2h_bytes_per_step": HEADLINE_BYTES, "ms_per_step": round(e2e_ms, 5),
                "nccl_value": None if e2e_nccl_ms is None else round(HEADLINE_BYTES / (e2e_nccl_ms * 1e-3) / 1e9, 3),
                "nccl_ms_per_step": None if e2e_nccl_ms is None else round(e2e_nccl_ms, 5)},
        "gpu_launches": int(launches),
        "nccl": None if nccl_ms is None else {"ms_per_step": round(nccl_ms, 5), "alg_bandwidth_GBps": round(HEADLINE_BYTES / nccl_ms / 1e6, 3)},
        "vs_nccl": None if nccl_ms is None else round(nccl_ms / ms_per_step, 4),
        "sweep": sweep,
        "sweep_variants": variants,
        "extras": extras,
        "cost_model": st["model"],
        "links": comm.topology().get("links"),
    }
    comm.destroy()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit_json(result)
    return 0 if not failures else 1


if __name__ == "__main__":
    sys.exit(main())
