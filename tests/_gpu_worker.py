"""One GPU rank (one process per GPU) of a multi-GPU scenario; see test_multigpu.py."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402

import cann_hccl_b200 as H  # noqa: E402
from cann_hccl_b200 import _lib as L  # noqa: E402


def make_comm(p, r, root_file):
    if r == 0:
        info = H.Communicator.get_root_info()
        with open(root_file + ".tmp", "wb") as f:
            f.write(info)
        os.rename(root_file + ".tmp", root_file)
    else:
        t0 = time.time()
        while not os.path.exists(root_file):
            assert time.time() - t0 < 60, "root info never appeared"
            time.sleep(0.01)
        with open(root_file, "rb") as f:
            info = f.read()
    cfg = L.CommConfig.default()
    cfg.hcclBufferSize = int(os.environ.get("TEST_BUFFSIZE_MB", "16"))
    return H.Communicator.init_root(p, info, r, config=cfg, device=True)


def inp(rank, n, dtype=torch.float32, seed=0):
    g = torch.Generator(device="cuda").manual_seed(1000 * seed + rank)
    if dtype.is_floating_point:
        return (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)
    return torch.randint(-3, 4, (n,), device="cuda", generator=g).to(dtype)


def red(xs, op):
    acc = xs[0].float() if xs[0].dtype in (torch.float16, torch.bfloat16) else xs[0].clone()
    for x in xs[1:]:
        y = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
        acc = {L.SUM: acc + y, L.PROD: acc * y, L.MAX: torch.maximum(acc, y), L.MIN: torch.minimum(acc, y)}[op]
    return acc.to(xs[0].dtype)


def close(a, b, dtype, p):
    if dtype == torch.float32:
        torch.testing.assert_close(a, b, rtol=2e-6 * p, atol=2e-6 * p)
    elif dtype in (torch.float16, torch.bfloat16):
        torch.testing.assert_close(a.float(), b.float(), rtol=1.6e-2, atol=1.6e-2 * p)
    else:
        assert torch.equal(a, b)


def ok(c):
    rc = c.sync()
    assert rc == 0, c.describe_status()


def scenario_collectives(c, p, r, args):
    nvls = c.has_nvls()
    print("rank %d: nvls=%s" % (r, nvls))
    ar_algos = [L.ALGO_AUTO, L.ALGO_LL, L.ALGO_MESH_ONESHOT, L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD, L.ALGO_MESH_PIPE] + ([L.ALGO_NVLS, L.ALGO_NVLS_ONESHOT, L.ALGO_NVLS_PIPE] if nvls else [])
    for n in (4, 1000, 262144, 6_000_000):  # the last one runs the staging loop (24 MB through 16 MB halves)
        for algo in ar_algos:
            if algo in (L.ALGO_NVLS, L.ALGO_NVLS_ONESHOT, L.ALGO_NVLS_PIPE) and (n * 4) % 16:
                continue
            if algo == L.ALGO_LL and n > 60000:
                continue
            for dtype, op in ((torch.float32, L.SUM), (torch.bfloat16, L.SUM), (torch.bfloat16, L.MAX), (torch.int32, L.MIN)):
                if algo in (L.ALGO_NVLS, L.ALGO_NVLS_ONESHOT, L.ALGO_NVLS_PIPE) and (n * dtype.itemsize) % 16:
                    continue
                if n > 1_000_000 and dtype != torch.float32:
                    continue
                xs = [inp(q, n, dtype, seed=n % 97) for q in range(p)]
                out = torch.zeros(n, device="cuda", dtype=dtype)
                c.all_reduce(xs[r], out, op=op, algo=algo)
                ok(c)
                try:
                    close(out, red(xs, op), dtype, p)
                except AssertionError as e:
                    bad = (out.float() - red(xs, op).float()).abs() > 1e-3
                    idx = bad.nonzero().flatten()
                    raise AssertionError("allreduce n=%d algo=%s dtype=%s op=%d: %d bad elements, first %d last %d\n%s" % (
                        n, L.ALGO_NAMES[algo], dtype, op, int(bad.sum()), int(idx[0]), int(idx[-1]), str(e)[:300]))
    if nvls:  # zero-copy on registered symmetric memory
        n = 2_000_000
        hin, (zin,) = c.symmetric_empty(n, torch.float32)
        hout, (zout,) = c.symmetric_empty(n, torch.float32)
        xs = [inp(q, n, torch.float32, seed=21) for q in range(p)]
        zin.copy_(xs[r])
        zout.zero_()
        c.all_reduce(zin, zout)
        ok(c)
        assert c.trace()[-1]["algo"] == ("nvls_zerocopy" if p > 2 else "mesh_zerocopy"), c.trace()[-1]
        close(zout, red(xs, L.SUM), torch.float32, p)
        c.all_reduce(zin, zin)  # in place
        ok(c)
        close(zin, red(xs, L.SUM), torch.float32, p)
        del zin, zout
        c.mem_free(hin)
        c.mem_free(hout)
    if nvls:  # tensors of the symmetric pool are ordinary torch tensors and run zero-copy without further calls
        n = 3_000_000
        pool = c.symmetric_pool()
        with torch.cuda.use_mem_pool(pool):
            pa = torch.empty(n, device="cuda")
            pb = torch.empty(n, device="cuda")
        xs = [inp(q, n, torch.float32, seed=23) for q in range(p)]
        pa.copy_(xs[r])
        c.all_reduce(pa, pb)
        ok(c)
        assert c.trace()[-1]["algo"] == ("nvls_zerocopy" if p > 2 else "mesh_zerocopy"), c.trace()[-1]
        close(pb, red(xs, L.SUM), torch.float32, p)
        del pa, pb
        torch.cuda.synchronize()
        c.barrier()
        ok(c)
        c.release_symmetric_pool()
    _adopted_vmm_memory(c, p, r, nvls)
    for algo in [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD] + ([L.ALGO_NVLS] if nvls else []):
        n = 40_000
        xs = [inp(q, n * p, torch.float32, seed=3) for q in range(p)]
        out = torch.zeros(n, device="cuda")
        c.reduce_scatter(xs[r], out, algo=algo)
        ok(c)
        close(out, red(xs, L.SUM)[r * n:(r + 1) * n], torch.float32, p)
        g = torch.zeros(n * p, device="cuda", dtype=torch.bfloat16)
        gs = [inp(q, n, torch.bfloat16, seed=4) for q in range(p)]
        c.all_gather(gs[r], g, algo=algo)
        ok(c)
        assert torch.equal(g, torch.cat(gs))
        if algo == L.ALGO_MESH:  # push variant
            g.zero_()
            c.all_gather(gs[r], g, algo=L.ALGO_PAIRWISE)
            ok(c)
            assert torch.equal(g, torch.cat(gs))
    # pipelined kernels on messages that go around the ring of staging slots several times (16 MB halves)
    pipes = [L.ALGO_MESH_PIPE] + ([L.ALGO_NVLS_PIPE] if nvls else [])
    for algo in pipes:
        for dtype in (torch.float32, torch.bfloat16):
            n = 1_500_000
            xs = [inp(q, n * p, dtype, seed=13) for q in range(p)]
            out = torch.zeros(n, device="cuda", dtype=dtype)
            c.reduce_scatter(xs[r], out, algo=algo)
            ok(c)
            close(out, red(xs, L.SUM)[r * n:(r + 1) * n], dtype, p)
            del xs
            gs = [inp(q, n, dtype, seed=14) for q in range(p)]
            g = torch.zeros(n * p, device="cuda", dtype=dtype)
            c.all_gather(gs[r], g, algo=algo)
            ok(c)
            assert torch.equal(g, torch.cat(gs))
            del gs, g
        for root in (0, p - 1):
            n = 9_000_000
            b = inp(r, n, torch.float32, seed=15)
            c.broadcast(b, root, algo=algo)
            ok(c)
            assert torch.equal(b, inp(root, n, torch.float32, seed=15))
        xs = [inp(q, 12_000_000, torch.float32, seed=16) for q in range(p)]
        want = red(xs, L.SUM)
        mine = xs[r].clone()
        for _ in range(3):  # back to back: staging halves alternate, counters are reused
            mine.copy_(xs[r])
            c.all_reduce(mine, mine, algo=algo)
        ok(c)
        close(mine, want, torch.float32, p)
        del xs, want, mine
    for root in (0, p - 1):
        for algo in [L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE] + ([L.ALGO_NVLS] if nvls else []):
            b = inp(r, 50_000, torch.float32, seed=5)
            c.broadcast(b, root, algo=algo)
            ok(c)
            assert torch.equal(b, inp(root, 50_000, torch.float32, seed=5))
        for algo in (L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE, L.ALGO_RHD):
            xs = [inp(q, 50_000, torch.float32, seed=6) for q in range(p)]
            out = torch.zeros(50_000, device="cuda")
            c.reduce(xs[r], out, root, algo=algo)
            ok(c)
            if r == root:
                close(out, red(xs, L.SUM), torch.float32, p)
    n = 3000
    for algo in (L.ALGO_MESH, L.ALGO_PAIRWISE):
        xs = [inp(q, n * p, torch.float32, seed=7) for q in range(p)]
        out = torch.zeros(n * p, device="cuda")
        c.all_to_all(xs[r], out, algo=algo)
        ok(c)
        for q in range(p):
            assert torch.equal(out[q * n:(q + 1) * n], xs[q][r * n:(r + 1) * n])
    # parametric AlltoAllV kernel (auto selection): uneven counts, blocks of several rounds, every rank its own row
    import numpy as np
    rng = np.random.default_rng(99)
    m = rng.integers(0, 900_000 // p, (p, p)).astype(np.uint64)
    m[0, p - 1] = 0
    sd = np.concatenate([[0], np.cumsum(m[r])[:-1]]).astype(np.uint64)
    rd = np.concatenate([[0], np.cumsum(m[:, r])[:-1]]).astype(np.uint64)
    rows = [inp(q, int(m[q].sum()) + 1, torch.float32, seed=17) for q in range(p)]
    vout = torch.zeros(int(m[:, r].sum()) + 1, device="cuda")
    for _ in range(2):
        c.all_to_all_v(rows[r], m[r].copy(), sd, vout, np.ascontiguousarray(m[:, r]), rd)
    ok(c)
    assert c.trace()[-1]["algo"] == "direct", c.trace()[-1]
    for q in range(p):
        sq = np.concatenate([[0], np.cumsum(m[q])[:-1]])
        assert torch.equal(vout[int(rd[q]):int(rd[q] + m[q, r])], rows[q][int(sq[r]):int(sq[r] + m[q, r])])
    c.barrier()
    ok(c)
    # Send/Recv ring over the NCCL p2p backend
    x = inp(r, 100_000, torch.float32, seed=8)
    y = torch.zeros_like(x)
    c.batch_send_recv([("send", x, (r + 1) % p), ("recv", y, (r - 1 + p) % p)])
    ok(c)
    assert torch.equal(y, inp((r - 1 + p) % p, 100_000, torch.float32, seed=8))
    if r % 2 == 0 and r + 1 < p:
        c.send(x, r + 1)
    elif r % 2 == 1:
        c.recv(y, r - 1)
        ok(c)
        assert torch.equal(y, inp(r - 1, 100_000, torch.float32, seed=8))
    ok(c)
    print("rank %d collectives ok; stats %s" % (r, c.stats()["algos"]))


def _adopted_vmm_memory(c, p, r, nvls):
    """User memory made with the driver's virtual-memory calls, registered through HcclCommSetMemoryRange /
    HcclCommActivateCommMemory: peers map it, put/get reach it, and AllReduce on it runs zero-copy."""
    try:
        from cuda.bindings import driver as drv
    except ImportError:
        print("rank %d: cuda-python missing, adopted-memory case skipped" % r)
        return
    import ctypes as C

    def chk(res):
        err, rest = res[0], res[1:]
        assert int(err) == 0, "driver call failed: %s" % err
        return rest[0] if len(rest) == 1 else rest

    dev = torch.cuda.current_device()
    prop = drv.CUmemAllocationProp()
    prop.type = drv.CUmemAllocationType.CU_MEM_ALLOCATION_TYPE_PINNED
    prop.location.type = drv.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    prop.location.id = dev
    prop.requestedHandleTypes = drv.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR
    size = 8 << 20
    acc = drv.CUmemAccessDesc()
    acc.location.type = drv.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    acc.location.id = dev
    acc.flags = drv.CUmemAccess_flags.CU_MEM_ACCESS_FLAGS_PROT_READWRITE
    regions = []
    for _ in range(2):  # send and receive buffer, one allocation each
        h = chk(drv.cuMemCreate(size, prop, 0))
        va = chk(drv.cuMemAddressReserve(size, 2 << 20, 0, 0))
        chk(drv.cuMemMap(va, size, 0, h, 0))
        chk(drv.cuMemSetAccess(va, size, [acc], 1))
        regions.append((int(h), int(va)))

    def view(va, n):
        class _P:
            pass
        o = _P()
        o.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (va, False), "version": 3}
        return torch.as_tensor(o, device="cuda")

    lib = L.lib()
    n = size // 4
    for h, va in regions:
        L.check(lib.HcclCommSetMemoryRange(c.handle, va, size, 0, 0), "HcclCommSetMemoryRange")
        L.check(lib.HcclCommActivateCommMemory(c.handle, va, size, 0, C.c_void_p(h), 0), "HcclCommActivateCommMemory")
    zin, zout = view(regions[0][1], n), view(regions[1][1], n)
    xs = [inp(q, n, torch.float32, seed=33) for q in range(p)]
    zin.copy_(xs[r])
    zout.zero_()
    c.all_reduce(zin, zout)
    ok(c)
    if nvls:
        assert c.trace()[-1]["algo"] == ("nvls_zerocopy" if p > 2 else "mesh_zerocopy"), c.trace()[-1]
    close(zout, red(xs, L.SUM), torch.float32, p)
    torch.cuda.synchronize()
    c.barrier()
    ok(c)
    for h, va in regions:
        L.check(lib.HcclCommDeactivateCommMemory(c.handle, va), "HcclCommDeactivateCommMemory")
        L.check(lib.HcclCommUnsetMemoryRange(c.handle, va), "HcclCommUnsetMemoryRange")
    zout.zero_()
    c.all_reduce(zin, zout)     # registration gone: staged path on the same memory
    ok(c)
    assert c.trace()[-1]["algo"] not in ("nvls_zerocopy", "mesh_zerocopy")
    close(zout, red(xs, L.SUM), torch.float32, p)
    torch.cuda.synchronize()
    del zin, zout
    for h, va in regions:
        chk(drv.cuMemUnmap(va, size))
        chk(drv.cuMemAddressFree(va, size))
        chk(drv.cuMemRelease(h))
    print("rank %d adopted vmm memory ok" % r)


def scenario_retry(c, p, r, args):
    """Operator retry on the device transport.  HCCL_FAULT_INJECT stalls rank 1 ON THE HOST before it launches its 2nd
    collective, for longer than the bound of the device waits: the peers' kernels give up (status block, no fault), the
    failure surfaces at the next synchronisation, all ranks vote over the hub and the op runs again."""
    n = 200_000
    for i in range(4):
        x = torch.full((n,), float(r + i), device="cuda")
        out = torch.zeros(n, device="cuda")
        c.all_reduce(x, out, algo=L.ALGO_MESH)
        rc = c.sync()
        assert rc == 0, (rc, c.describe_status())
        assert torch.all(out == float(sum(q + i for q in range(p)))), "allreduce %d wrong after retry" % i
    st = c.stats()
    print("rank %d retries %d timeouts %d" % (r, st["retries"], st["timeouts"]))
    assert st["retries"] >= 1
    print("rank %d retry ok" % r)


def scenario_retry_exhausted(c, p, r, args):
    """The stall also hits every retry: after the configured number of attempts the failure is returned, and the
    communicator works again once it has been resumed."""
    n = 50_000
    x = torch.full((n,), float(r), device="cuda")
    out = torch.zeros(n, device="cuda")
    c.all_reduce(x, out, algo=L.ALGO_MESH)
    assert c.sync() == 0
    try:
        c.all_reduce(x, out, algo=L.ALGO_MESH)  # op 2: stalled on rank 1, and again on each retry
        rc = c.sync()                           # the rank whose kernels gave up learns it here ...
    except H.HcclError as e:
        rc = e.code                             # ... the stalled rank joined the retry rounds from inside the call
    assert rc in (L.E_TIMEOUT, L.E_REMOTE), rc
    assert c.stats()["retries"] == 3, c.stats()
    c.resume()
    out.zero_()
    c.all_reduce(x, out, algo=L.ALGO_MESH)
    assert c.sync() == 0, c.describe_status()
    assert torch.all(out == float(sum(range(p))))
    print("rank %d retry exhausted ok" % r)


def scenario_fused_tp(c, p, r, args):
    """Fused all-gather+GEMM and GEMM+reduce-scatter across real GPUs against the fp32 PyTorch statement."""
    from cann_hccl_b200.parallel import fused_tp
    Ms, K, N = 256, 1024, 768
    g = lambda q, shape, seed, scale=1.0: (torch.randn(*shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(100 * seed + q)) * scale).to(torch.bfloat16)
    xs = [g(q, (Ms, K), 1) for q in range(p)]
    w = g(r, (N, K), 2, 0.05)
    for _ in range(4):
        y = fused_tp.all_gather_matmul(c, xs[r], w)
        ok(c)
    ref = torch.cat([x.float() for x in xs]) @ w.float().t()
    err = float((y.float() - ref).norm() / ref.norm())
    assert err < 1e-2, err
    # the same with the shard in registered symmetric memory: peers pull it in place, and it may be rewritten after the call
    handle, bufs = c.symmetric_empty(Ms * K, torch.bfloat16)
    xz = bufs[0].view(Ms, K)
    for _ in range(3):
        xz.copy_(xs[r])
        y = fused_tp.all_gather_matmul(c, xz, w)
        xz.zero_()
        ok(c)
        err = float((y.float() - ref).norm() / ref.norm())
        assert err < 1e-2, err
    M = Ms * p
    hs = [g(q, (M, K), 3) for q in range(p)]
    ws = [g(q, (N, K), 4, 0.05) for q in range(p)]
    for _ in range(4):
        o = fused_tp.matmul_reduce_scatter(c, hs[r], ws[r])
        ok(c)
    full = sum(hq.float() @ wq.float().t() for hq, wq in zip(hs, ws))
    err = float((o.float() - full[r * Ms:(r + 1) * Ms]).norm() / full.norm())
    assert err < 2e-2, err
    print("rank %d fused_tp ok" % r)


if __name__ == "__main__":
    scenario, p, r, root_file = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    torch.cuda.set_device(r)
    comm = make_comm(p, r, root_file)
    globals()["scenario_" + scenario](comm, p, r, sys.argv[5:])
    assert comm.destroy() == L.SUCCESS
