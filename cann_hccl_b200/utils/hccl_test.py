"""hccl_test-shaped command line: sweep one collective over message sizes and print, per size, the columns of the
reference's external HCCL-Test tool (its README: `mpirun -n 8 ./bin/all_reduce_test -b 8K -e 64M -f 2 -d fp32 -o sum -p 8`,
output `data_size`, `aveg_time` us, `alg_bandwidth` GB/s, `check_result`).

    python -m cann_hccl_b200.utils.hccl_test all_reduce_test -b 8K -e 64M -f 2 -d fp32 -o sum -p 8
    python -m cann_hccl_b200.utils.hccl_test all_gather_test -b 1K -e 1M -f 4 -d int32 -p 4 --host     # CPU ranks
    python -m cann_hccl_b200.utils.hccl_test all_reduce_test -b 1M -e 1G -p 8 --algo mesh_pipe,nvls_pipe --nccl --trace

`--algo` takes one algorithm or a comma-separated list (one timed column per name after the selector's own choice),
`--nccl` adds the same collective through torch.distributed's NCCL backend on the same buffers, `--trace` prints the
in-kernel stage times of the newest pipelined launch of rank 0 (wait / work / publish per stage, microseconds).

One process per rank is started by this program itself (no mpirun): rank 0 writes the root info to a temporary file, the
others read it.  On GPUs rank r uses device r; the timed calls are issued back to back from C and timed with CUDA events
(host transport: wall clock), `aveg_time` is the maximum over ranks.  `check_result` compares every rank's output with the
numpy reference built from the seeded inputs of all ranks (uniform[-1,1) floats / small integers, seed 1234 + rank).

Tests: all_reduce_test, all_gather_test, reduce_scatter_test, broadcast_test, reduce_test, scatter_test, gather_test,
alltoall_test.  `-b/-e` are bytes per rank of the collective's `count` argument times the element size (the send count for
all_gather / gather / alltoall, the receive count for reduce_scatter / scatter).
"""
import argparse
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

TESTS = ("all_reduce_test", "all_gather_test", "reduce_scatter_test", "broadcast_test", "reduce_test", "scatter_test", "gather_test",
         "alltoall_test", "alltoallv_test")
NP_DTYPES = {"int8": np.int8, "uint8": np.uint8, "int16": np.int16, "uint16": np.uint16, "int32": np.int32, "uint32": np.uint32,
             "int64": np.int64, "uint64": np.uint64, "fp16": np.float16, "fp32": np.float32, "fp64": np.float64, "bfp16": None}
OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3}


def parse_size(s):
    s = s.strip().upper()
    mult = 1
    if s[-1] in "KMG":
        mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}[s[-1]]
        s = s[:-1]
    return int(float(s) * mult)


def make_input(rank, n, dtype_name, seed_base=1234):
    """Seeded input of one rank as a numpy array (bfp16 is produced as float32 values that are exact in bfloat16)."""
    rng = np.random.default_rng(seed_base + rank)
    if dtype_name in ("fp16", "fp32", "fp64", "bfp16"):
        x = rng.uniform(-1, 1, n).astype(np.float32)
        if dtype_name == "bfp16":
            x = (x.view(np.uint32) & np.uint32(0xFFFF0000)).view(np.float32)
            return x
        return x.astype(NP_DTYPES[dtype_name])
    return rng.integers(0, 3, n).astype(NP_DTYPES[dtype_name])


def reference(test, ins, op, p, rank, root, count):
    """numpy result of rank `rank` (None when the rank receives nothing)."""
    def red(arrs):
        acc = arrs[0].astype(np.float64) if arrs[0].dtype.kind == "f" else arrs[0].copy()
        for a in arrs[1:]:
            b = a.astype(np.float64) if a.dtype.kind == "f" else a
            acc = {0: acc + b, 1: acc * b, 2: np.maximum(acc, b), 3: np.minimum(acc, b)}[op]
        return acc
    if test == "all_reduce_test":
        return red(ins)
    if test == "reduce_test":
        return red(ins) if rank == root else None
    if test == "all_gather_test":
        return np.concatenate(ins)
    if test == "gather_test":
        return np.concatenate(ins) if rank == root else None
    if test == "reduce_scatter_test":
        return red(ins)[rank * count:(rank + 1) * count]
    if test == "broadcast_test":
        return ins[root]
    if test == "scatter_test":
        return ins[root][rank * count:(rank + 1) * count]
    if test == "alltoall_test":
        return np.concatenate([ins[q][rank * count:(rank + 1) * count] for q in range(p)])
    if test == "alltoallv_test":
        m = a2av_matrix(count, p)
        return np.concatenate([ins[q][int(m[q, :rank].sum()):int(m[q, :rank + 1].sum())] for q in range(p)])
    raise ValueError(test)


def a2av_matrix(count, p):
    """Count matrix of alltoallv_test: rank i sends count * ((i + j) % 4 + 1) / 4 elements to rank j (at least one)."""
    return np.array([[max(1, count * ((i + j) % 4 + 1) // 4) for j in range(p)] for i in range(p)], dtype=np.uint64)


def a2av_rows(m, ranks):
    """(send counts, send displacements, receive counts, receive displacements) of the listed ranks, one row per rank."""
    sc = np.stack([m[r] for r in ranks])
    rc = np.stack([m[:, r] for r in ranks])
    excl = lambda c: np.concatenate([np.zeros((c.shape[0], 1), np.uint64), np.cumsum(c, axis=1)[:, :-1]], axis=1).astype(np.uint64)
    return sc, excl(sc), rc, excl(rc)


def in_elems(test, count, p):
    return count * p if test in ("reduce_scatter_test", "scatter_test", "alltoall_test") else count


def out_elems(test, count, p):
    return count * p if test in ("all_gather_test", "gather_test", "alltoall_test") else count


def worker(a):
    rank, p = a.rank, a.nranks
    if a.host:
        os.environ["HCCL_TRANSPORT"] = "host"
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    import cann_hccl_b200 as H
    from cann_hccl_b200 import _lib as L
    device = not a.host
    local = bool(a.local)  # every rank a virtual rank of this process's GPU: one cooperative launch per collective
    torch = None
    if device:
        import torch
        torch.cuda.set_device(rank % torch.cuda.device_count())
    # rendezvous through a file
    if local:
        info = None
    elif rank == 0:
        info = H.Communicator.get_root_info()
        with open(a.root_file + ".tmp", "wb") as f:
            f.write(info)
        os.rename(a.root_file + ".tmp", a.root_file)
    else:
        t0 = time.time()
        while not os.path.exists(a.root_file):
            if time.time() - t0 > 60:
                raise RuntimeError("root info never appeared")
            time.sleep(0.01)
        info = open(a.root_file, "rb").read()
    cfg = L.CommConfig.default()
    cfg.hcclBufferSize = a.buffsize
    if local:
        comm = H.Communicator.init_local(p, device=True, device_id=torch.cuda.current_device(), config=cfg)
    else:
        comm = H.Communicator.init_root(p, info, rank, config=cfg, device=device)
    coll = {"all_reduce_test": L.ALLREDUCE, "all_gather_test": L.ALLGATHER, "reduce_scatter_test": L.REDUCE_SCATTER, "broadcast_test": L.BROADCAST,
            "reduce_test": L.REDUCE, "scatter_test": L.SCATTER, "gather_test": L.GATHER, "alltoall_test": L.ALLTOALL, "alltoallv_test": L.ALLTOALLV}[a.test]
    hd = {"int8": L.INT8, "uint8": L.UINT8, "int16": L.INT16, "uint16": L.UINT16, "int32": L.INT32, "uint32": L.UINT32, "int64": L.INT64,
          "uint64": L.UINT64, "fp16": L.FP16, "fp32": L.FP32, "fp64": L.FP64, "bfp16": L.BFP16}[a.dtype]
    es = 2 if a.dtype == "bfp16" else np.dtype(NP_DTYPES[a.dtype]).itemsize
    op = OPS[a.op]
    names = [x for x in a.algo.split(",") if x] if a.algo else []
    for x in names:
        if x not in L.ALGO_NAMES:
            raise SystemExit("unknown algorithm %r (known: %s)" % (x, ", ".join(L.ALGO_NAMES)))
    # one name: that algorithm replaces the selector (as before); several: the selector's choice first, then a column each
    algo = L.ALGO_NAMES.index(names[0]) if len(names) == 1 else L.ALGO_AUTO
    extra_algos = names if len(names) > 1 else []
    dist = None
    if a.nccl and device and p > 1 and not local:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29600 + (os.getppid() % 300)))
        dist.init_process_group("nccl", rank=rank, world_size=p, device_id=torch.device("cuda", torch.cuda.current_device()))
    if rank == 0:
        print("the minbytes is %d, maxbytes is %d, iters is %d, warmup_iters is %d" % (a.minbytes, a.maxbytes, a.iters, a.warmup))
        head = "%-16s %-16s %-22s %-14s" % ("data_size(Bytes):", "aveg_time(us):", "alg_bandwidth(GB/s):", "check_result:")
        head += "".join(" %-16s" % (x + "(us):") for x in extra_algos) + (" %-16s %-16s" % ("nccl_time(us):", "nccl_bw(GB/s):") if dist else "")
        print(head)
    size = a.minbytes
    failed = False
    while size <= a.maxbytes:
        count = max(1, size // es)
        v = a.test == "alltoallv_test"
        mat = a2av_matrix(count, p) if v else None
        n_in_of = (lambda q: int(mat[q].sum())) if v else (lambda q: in_elems(a.test, count, p))
        n_out_of = (lambda q: int(mat[:, q].sum())) if v else (lambda q: out_elems(a.test, count, p))
        n_in, n_out = n_in_of(rank), n_out_of(rank)
        mine = make_input(rank, n_in, a.dtype)
        if local:
            tdt = {"bfp16": torch.bfloat16}.get(a.dtype)
            send = [torch.from_numpy(make_input(q, n_in_of(q), a.dtype)).cuda() for q in range(p)]
            send = [x.to(tdt) for x in send] if tdt else send
            recv = send if a.test == "broadcast_test" else [torch.zeros(n_out_of(q), device="cuda", dtype=send[0].dtype) for q in range(p)]
        elif device:
            tdt = {"bfp16": torch.bfloat16}.get(a.dtype)
            send = torch.from_numpy(mine).cuda().to(tdt) if tdt else torch.from_numpy(mine).cuda()
            recv = send if a.test == "broadcast_test" else torch.zeros(n_out, device="cuda", dtype=send.dtype)
        else:
            if a.dtype == "bfp16":
                send = (mine.view(np.uint32) >> 16).astype(np.uint16)  # bf16 bit patterns
            else:
                send = mine
            recv = send if a.test == "broadcast_test" else np.zeros(n_out, send.dtype)
        kw = dict(op=op, root=a.root, algo=algo)

        rows = a2av_rows(mat, range(p) if local else [rank]) if v else None

        def call(k, **over):
            if k <= 0:
                return
            if v:  # the count matrix travels with every call: a Python loop instead of the C loop
                for _ in range(k):
                    comm.all_to_all_v(send, rows[0], rows[1], recv, rows[2], rows[3], algo=dict(kw, **over)["algo"])
            else:
                comm.repeat(coll, send, recv, count, hd, k, **dict(kw, **over))

        # one checked call, then warm-up and the timed loop
        call(1)
        if device:
            assert comm.sync() == 0, comm.describe_status()
        ok = True
        if a.check:
            ins = [make_input(q, n_in_of(q), a.dtype) for q in range(p)]
            for vr, got_t in (enumerate(recv) if local else ((rank, recv),)):
                ref = reference(a.test, ins, op, p, vr, a.root, count)
                if ref is None:
                    continue
                if device:
                    got = got_t.float().cpu().numpy() if a.dtype in ("bfp16", "fp16") else got_t.cpu().numpy()
                elif a.dtype == "bfp16":
                    got = (got_t.astype(np.uint32) << 16).view(np.float32)
                else:
                    got = got_t
                if np.asarray(ref).dtype.kind == "f" or got.dtype.kind == "f":
                    tol = {"fp64": 1e-12, "fp32": 1e-5, "fp16": 4e-3, "bfp16": 2e-2}.get(a.dtype, 1e-5) * max(1, p // 2)
                    ok = ok and bool(np.allclose(got.astype(np.float64), np.asarray(ref, np.float64), rtol=tol, atol=tol))
                else:
                    ok = ok and bool(np.array_equal(got, ref.astype(got.dtype)))
        def timed(fn):
            fn(a.warmup)
            if not local:
                comm.barrier()
            if device:
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn(a.iters)
                e1.record()
                torch.cuda.synchronize()
                assert comm.sync() == 0, comm.describe_status()
                return e0.elapsed_time(e1) * 1e3 / a.iters
            t0 = time.perf_counter()
            fn(a.iters)
            return (time.perf_counter() - t0) * 1e6 / a.iters
        times = [timed(call)]
        notes = []

        def stage_times(label):
            """In-kernel stage times of the newest launch when that was a pipelined kernel (its trace has another layout)."""
            if not (a.trace and rank == 0 and device):
                return
            last = comm.trace()[-1]["algo"]
            text = "    %s ran %s" % (label, last)
            if last in ("mesh_pipe", "nvls_pipe", "mesh_zerocopy"):
                import ctypes as C
                buf = (C.c_uint64 * 16)()
                ns = C.c_int(0)
                if L.lib().HcclB200GetKernelTrace(comm.handle, 0, buf, 16, C.byref(ns)) == 0 and buf[0] not in (0, 2 ** 64 - 1):
                    text += "; stage times of its newest launch (us): " + " | ".join(
                        "stage %d wait %.1f work %.1f publish %.1f" % (k, buf[1 + 4 * k] / 1e3, buf[2 + 4 * k] / 1e3, buf[3 + 4 * k] / 1e3) for k in range(3))
            notes.append(text)
        stage_times("the selector's choice:")
        for x in extra_algos:
            kx = dict(kw, algo=L.ALGO_NAMES.index(x))
            try:
                times.append(timed(lambda k: call(k, algo=kx["algo"])))
                stage_times("forced %s:" % x)
            except H.HcclError:
                times.append(float("nan"))  # the algorithm does not exist for this collective / type / size
        if dist is not None:
            nccl_fn = {"all_reduce_test": lambda: dist.all_reduce(recv if recv is not send else send, op={0: dist.ReduceOp.SUM, 1: dist.ReduceOp.PRODUCT, 2: dist.ReduceOp.MAX, 3: dist.ReduceOp.MIN}[op]),
                       "all_gather_test": lambda: dist.all_gather_into_tensor(recv, send),
                       "reduce_scatter_test": lambda: dist.reduce_scatter_tensor(recv, send),
                       "broadcast_test": lambda: dist.broadcast(send, src=a.root),
                       "reduce_test": lambda: dist.reduce(send, dst=a.root),
                       "scatter_test": lambda: dist.scatter(recv, list(send.chunk(p)) if rank == a.root else None, src=a.root),
                       "gather_test": lambda: dist.gather(send, list(recv.chunk(p)) if rank == a.root else None, dst=a.root),
                       "alltoall_test": lambda: dist.all_to_all_single(recv, send),
                       "alltoallv_test": lambda: dist.all_to_all_single(recv, send, [int(x) for x in mat[:, rank]], [int(x) for x in mat[rank]])}[a.test]
            times.append(timed(lambda k: [nccl_fn() for _ in range(k)]))
        # maximum over ranks and the conjunction of the checks, gathered over the control plane
        import struct
        fmt = "<%ddI" % len(times)
        mine_blob = struct.pack(fmt, *times, 1 if ok else 0)
        blob = [mine_blob] if local else comm.exchange("t%d" % size, mine_blob)
        vals = [struct.unpack(fmt, b) for b in blob]
        times = [max(v[i] for v in vals) for i in range(len(times))]
        us = times[0]
        ok = all(v[-1] for v in vals)
        failed |= not ok
        if rank == 0:
            line = "%-16d %-16.2f %-22.5f %-14s" % (count * es, us, count * es / us / 1e3, "success" if ok else "failed")
            line += "".join(" %-16.2f" % t for t in times[1:1 + len(extra_algos)])
            if dist is not None:
                line += " %-16.2f %-16.5f" % (times[-1], count * es / times[-1] / 1e3)
            print(line, flush=True)
            for t in notes:
                print(t, flush=True)
        del send, recv
        size = size * a.factor if a.factor > 1 else size + max(1, a.step)
    code = comm.destroy()
    if dist is not None:
        dist.destroy_process_group()
    return 1 if failed or code != 0 else 0


def main(argv=None):
    ap = argparse.ArgumentParser(prog="hccl_test", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("test", choices=TESTS)
    ap.add_argument("-b", "--minbytes", default="8K")
    ap.add_argument("-e", "--maxbytes", default="64M")
    ap.add_argument("-f", "--factor", type=int, default=2, help="multiply the size by this each step (0/1: use -i)")
    ap.add_argument("-i", "--step", type=int, default=0, help="size increment in bytes when -f is 0 or 1")
    ap.add_argument("-d", "--dtype", default="fp32", choices=sorted(NP_DTYPES))
    ap.add_argument("-o", "--op", default="sum", choices=sorted(OPS))
    ap.add_argument("-p", "--nranks", type=int, default=0, help="ranks (default: visible GPUs, or 2 with --host)")
    ap.add_argument("-n", "--iters", type=int, default=20)
    ap.add_argument("-w", "--warmup", type=int, default=5)
    ap.add_argument("-c", "--check", type=int, default=1)
    ap.add_argument("-r", "--root", type=int, default=0)
    ap.add_argument("--algo", default="", help="force an algorithm (mesh, ring, rhd, nvls, ...); a comma-separated list adds one timed column per name")
    ap.add_argument("--nccl", action="store_true", help="also time the same collective through torch.distributed (NCCL) on the same buffers")
    ap.add_argument("--trace", action="store_true", help="print the in-kernel stage times of the newest pipelined launch (sets HCCL_KERNEL_TRACE=1)")
    ap.add_argument("--host", action="store_true", help="CPU ranks over the host-memory transport")
    ap.add_argument("--local", action="store_true", help="all ranks as virtual ranks of ONE GPU in one process (one cooperative launch per "
                    "collective); chosen automatically when -p asks for more ranks than GPUs are visible")
    ap.add_argument("--buffsize", type=int, default=200, help="staging MB per direction (HCCL_BUFFSIZE)")
    ap.add_argument("--rank", type=int, default=-1, help=argparse.SUPPRESS)
    ap.add_argument("--root-file", default="", help=argparse.SUPPRESS)
    a = ap.parse_args(argv)
    a.minbytes, a.maxbytes = parse_size(a.minbytes), parse_size(a.maxbytes)
    os.environ.setdefault("HCCL_EXEC_TIMEOUT_MS", "30000")  # a lost rank must not leave the others' waits polling for long
    if a.trace:
        os.environ["HCCL_KERNEL_TRACE"] = "1"
    if a.rank >= 0:
        return worker(a)
    if a.nranks <= 0:
        if a.host:
            a.nranks = 2
        else:
            import torch
            a.nranks = max(1, torch.cuda.device_count())
    if not a.host:
        import torch
        # kernels of different ranks wait on one another, so ranks never share a GPU as separate processes
        if a.local or a.nranks > torch.cuda.device_count():
            a.local, a.rank = True, 0
            return worker(a)
    tmp = tempfile.mkdtemp(prefix="hccl_test_")
    root_file = os.path.join(tmp, "root.bin")
    base = [sys.executable, "-m", "cann_hccl_b200.utils.hccl_test"] + [x for x in (argv if argv is not None else sys.argv[1:])]
    if "-p" not in base and "--nranks" not in base:
        base += ["-p", str(a.nranks)]
    env = dict(os.environ)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    procs = [subprocess.Popen(base + ["--rank", str(r), "--root-file", root_file], env=env) for r in range(a.nranks)]
    codes = [p.wait() for p in procs]
    return 0 if all(c == 0 for c in codes) else 1


if __name__ == "__main__":
    sys.exit(main())
