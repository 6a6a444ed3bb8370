"""One CPU rank of a multi-process scenario (see mp_util.run_ranks)."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import ctypes as C  # noqa: E402
import numpy as np  # noqa: E402

import cann_hccl_b200 as H  # noqa: E402
from cann_hccl_b200 import _lib as L  # noqa: E402
from oracle import np_reduce  # noqa: E402


def make_comm(nranks, rank, root_file, config=None):
    if rank == 0:
        info = H.Communicator.get_root_info()
        with open(root_file + ".tmp", "wb") as f:
            f.write(info)
        os.rename(root_file + ".tmp", root_file)
    else:
        t0 = time.time()
        while not os.path.exists(root_file):
            if time.time() - t0 > 30:
                raise RuntimeError("root info never appeared")
            time.sleep(0.01)
        with open(root_file, "rb") as f:
            info = f.read()
    return H.Communicator.init_root(nranks, info, rank, config=config, device=False)


def rank_input(rank, n, dtype=np.float32):
    return np.random.default_rng(1234 + rank).uniform(-1, 1, n).astype(dtype)


def scenario_allreduce_ring_8mb(c, p, r, args):
    """BASELINE config (a): AllReduce sum fp32, 2,097,152 elements per rank, Ring, rtol 1e-6."""
    n = 2_097_152
    x = rank_input(r, n)
    out = np.zeros_like(x)
    t0 = time.time()
    c.all_reduce(x, out, algo=L.ALGO_RING)
    dt = time.time() - t0
    ref = np_reduce([rank_input(q, n) for q in range(p)], L.SUM)
    np.testing.assert_allclose(out, ref, rtol=1e-6, atol=1e-6)
    print("check_result: success  aveg_time(us): %.1f  alg_bandwidth(GB/s): %.3f  data_size: %d" % (dt * 1e6, n * 4 / dt / 1e9, n * 4))


def scenario_a2av_mismatch(c, p, r, args):
    """Rank 1 expects one element more from rank 0 than rank 0 sends: every rank gets HCCL_E_PARA, nothing hangs; a
    consistent call afterwards works."""
    lib = L.lib()
    sc = np.full(p, 4, np.uint64)
    rcnt = np.full(p, 4, np.uint64)
    if r == 1:
        rcnt[0] = 5
    sd = np.arange(p, dtype=np.uint64) * 4
    rd = np.arange(p, dtype=np.uint64) * 8
    x = np.full(4 * p, float(r), np.float32)
    y = np.zeros(8 * p, np.float32)
    rc = lib.HcclAlltoAllV(x.ctypes.data, sc.ctypes.data, sd.ctypes.data, L.FP32, y.ctypes.data, rcnt.ctypes.data, rd.ctypes.data, L.FP32, c.handle, None)
    assert rc == L.E_PARA, rc
    rcnt[:] = 4
    rc = lib.HcclAlltoAllV(x.ctypes.data, sc.ctypes.data, sd.ctypes.data, L.FP32, y.ctypes.data, rcnt.ctypes.data, rd.ctypes.data, L.FP32, c.handle, None)
    assert rc == 0, rc
    for q in range(p):
        np.testing.assert_array_equal(y[q * 8:q * 8 + 4], np.full(4, float(q), np.float32))
    print("a2av_mismatch ok")


def scenario_sweep(c, p, r, args):
    n = 10_000
    for algo in (L.ALGO_AUTO, L.ALGO_MESH, L.ALGO_MESH_ONESHOT, L.ALGO_RING, L.ALGO_RHD):
        x = rank_input(r, n)
        out = np.zeros_like(x)
        c.all_reduce(x, out, algo=algo)
        np.testing.assert_allclose(out, np_reduce([rank_input(q, n) for q in range(p)], L.SUM), rtol=1e-5, atol=1e-5)
    # C API entry points with HCCL signatures
    lib = L.lib()
    x = rank_input(r, n)
    g = np.zeros(n * p, np.float32)
    L.check(lib.HcclAllGather(x.ctypes.data, g.ctypes.data, n, L.FP32, c.handle, None), "HcclAllGather")
    np.testing.assert_array_equal(g, np.concatenate([rank_input(q, n) for q in range(p)]))
    rs = np.zeros(n // p, np.float32)
    L.check(lib.HcclReduceScatter(x.ctypes.data, rs.ctypes.data, n // p, L.FP32, L.SUM, c.handle, None), "HcclReduceScatter")
    full = np_reduce([rank_input(q, n) for q in range(p)], L.SUM)
    np.testing.assert_allclose(rs, full[r * (n // p):(r + 1) * (n // p)], rtol=1e-5, atol=1e-5)
    b = rank_input(r, 100)
    L.check(lib.HcclBroadcast(b.ctypes.data, 100, L.FP32, 1 % p, c.handle, None), "HcclBroadcast")
    np.testing.assert_array_equal(b, rank_input(1 % p, 100))
    red = np.zeros(n, np.float32)
    L.check(lib.HcclReduce(x.ctypes.data, red.ctypes.data, n, L.FP32, L.MAX, 0, c.handle, None), "HcclReduce")
    if r == 0:
        np.testing.assert_array_equal(red, np_reduce([rank_input(q, n) for q in range(p)], L.MAX))
    sc = np.zeros(10, np.float32)
    src = np.arange(10 * p, dtype=np.float32)
    L.check(lib.HcclScatter(src.ctypes.data, sc.ctypes.data, 10, L.FP32, 0, c.handle, None), "HcclScatter")
    np.testing.assert_array_equal(sc, src[r * 10:(r + 1) * 10])
    ga = np.zeros(10 * p, np.float32)
    mine = np.full(10, r, np.float32)
    L.check(lib.HcclGather(mine.ctypes.data, ga.ctypes.data, 10, L.FP32, p - 1, c.handle, None), "HcclGather")
    if r == p - 1:
        np.testing.assert_array_equal(ga, np.repeat(np.arange(p, dtype=np.float32), 10))
    a2a_in = np.arange(p * 4, dtype=np.float32) + 100 * r
    a2a_out = np.zeros(p * 4, np.float32)
    L.check(lib.HcclAlltoAll(a2a_in.ctypes.data, 4, L.FP32, a2a_out.ctypes.data, 4, L.FP32, c.handle, None), "HcclAlltoAll")
    for q in range(p):
        np.testing.assert_array_equal(a2a_out[q * 4:(q + 1) * 4], np.arange(r * 4, r * 4 + 4) + 100 * q)
    # AlltoAllV: rank i sends (i + j + 1) elements to rank j
    scnt = np.array([r + j + 1 for j in range(p)], np.uint64)
    rcnt = np.array([j + r + 1 for j in range(p)], np.uint64)
    sdis = np.concatenate([[0], np.cumsum(scnt)[:-1]]).astype(np.uint64)
    rdis = np.concatenate([[0], np.cumsum(rcnt)[:-1]]).astype(np.uint64)
    vin = np.concatenate([np.full(int(scnt[j]), 10 * r + j, np.float32) for j in range(p)])
    vout = np.zeros(int(rcnt.sum()), np.float32)
    L.check(lib.HcclAlltoAllV(vin.ctypes.data, scnt.ctypes.data, sdis.ctypes.data, L.FP32, vout.ctypes.data, rcnt.ctypes.data,
                              rdis.ctypes.data, L.FP32, c.handle, None), "HcclAlltoAllV")
    for j in range(p):
        np.testing.assert_array_equal(vout[int(rdis[j]):int(rdis[j] + rcnt[j])], np.full(int(rcnt[j]), 10 * j + r, np.float32))
    # AlltoAllVC with the full matrix
    m = np.array([[i + j + 1 for j in range(p)] for i in range(p)], np.uint64)
    vout[:] = 0
    L.check(lib.HcclAlltoAllVC(vin.ctypes.data, m.ctypes.data, L.FP32, vout.ctypes.data, L.FP32, c.handle, None), "HcclAlltoAllVC")
    for j in range(p):
        np.testing.assert_array_equal(vout[int(rdis[j]):int(rdis[j] + rcnt[j])], np.full(int(rcnt[j]), 10 * j + r, np.float32))
    L.check(lib.HcclBarrier(c.handle, None), "HcclBarrier")
    print("sweep ok")


def scenario_sendrecv(c, p, r, args):
    n = 200_000  # 800 KB: several mailbox rounds
    right, left = (r + 1) % p, (r - 1 + p) % p
    x = rank_input(r, n)
    y = np.zeros_like(x)
    if r % 2 == 0:
        c.send(x, right)
        c.recv(y, left)
    else:
        c.recv(y, left)
        c.send(x, right)
    np.testing.assert_array_equal(y, rank_input(left, n))
    # batch: ring exchange in both directions + a self pair
    y2, z2, s2 = np.zeros_like(x), np.zeros_like(x), np.zeros(8, np.float32)
    me = np.full(8, r, np.float32)
    c.batch_send_recv([("recv", y2, left), ("send", x, right), ("send", x, left), ("recv", z2, right),
                       ("send", me, r), ("recv", s2, r)])
    np.testing.assert_array_equal(y2, rank_input(left, n))
    np.testing.assert_array_equal(z2, rank_input(right, n))
    np.testing.assert_array_equal(s2, me)
    print("sendrecv ok")


def scenario_subcomm(c, p, r, args):
    # even ranks form a sub-communicator, odd ranks stay out
    members = list(range(0, p, 2))
    sub = c.create_sub(members, 7, members.index(r) if r in members else None)
    if r in members:
        assert sub is not None and sub.nranks == len(members) and sub.rank == members.index(r)
        assert sub.name().endswith("_sub_7")
        x = np.full(100, r + 1, np.float32)
        out = np.zeros_like(x)
        sub.all_reduce(x, out)
        np.testing.assert_array_equal(out, np.full(100, sum(m + 1 for m in members), np.float32))
        assert sub.destroy() == L.SUCCESS
    else:
        assert sub is None
    x = np.full(10, 1, np.float32)
    out = np.zeros_like(x)
    c.all_reduce(x, out)
    np.testing.assert_array_equal(out, np.full(10, p, np.float32))
    print("subcomm ok")


def scenario_hcom(c, p, r, args):
    """Group-name front end: world group adopted from a communicator, a group over the odd ranks, rank translation,
    gradient fusion settings and the bucketed data-parallel AllReduce that reads them."""
    from cann_hccl_b200.ops import hcom
    from cann_hccl_b200.parallel import grad_bucket
    hcom.init_by_comm(c)
    assert hcom.rank_size() == p and hcom.rank_id() == r
    members = list(range(1, p, 2))
    hcom.create_group("odd", members)
    assert hcom.rank_size("odd") == len(members)
    assert hcom.world_rank_from_group_rank("odd", 0) == 1
    assert hcom.group_rank_from_world_rank(members[-1], "odd") == len(members) - 1
    sub = hcom.group_comm("odd")
    if r in members:
        assert sub is not None and sub.rank == members.index(r) and hcom.rank_id("odd") == sub.rank
        x = np.full(64, r, np.float32)
        out = np.zeros_like(x)
        sub.all_reduce(x, out)
        np.testing.assert_array_equal(out, np.full(64, sum(members), np.float32))
    else:
        assert sub is None
    lib = L.lib()
    bad = (L.C.c_uint32 * 2)(3, 3)
    assert lib.HcomSetGradFusionByIndex(None, 2, bad) == L.E_PARA            # not ascending
    shares = (L.C.c_float * 2)(30.0, 60.0)
    assert lib.HcomSetGradFusionBySize(None, 2, shares) == L.E_PARA         # does not sum to 100
    assert hcom.grad_fusion_by_index() is None
    # three segments by index over seven gradients: [0..1], [2..4], [5..6]
    hcom.set_grad_fusion_by_index(None, [1, 4, 6])
    shapes = [(5,), (3, 4), (7,), (2, 2), (9,), (1,), (6,)]
    grads = [np.random.default_rng(100 * q + r).uniform(-1, 1, sh).astype(np.float32) for q, sh in enumerate(shapes)]
    want = [sum(np.random.default_rng(100 * q + rr).uniform(-1, 1, sh).astype(np.float32) for rr in range(p)) / p for q, sh in enumerate(shapes)]
    calls = lambda: c.stats()["ops"].get("AllReduce", {"calls": 0})["calls"]
    before = calls()
    segs = grad_bucket.all_reduce_gradients(c, grads)
    assert segs == [(0, 2), (2, 5), (5, 7)], segs
    assert calls() - before == 3
    for g, w in zip(grads, want):
        np.testing.assert_allclose(g, w, rtol=1e-5, atol=1e-6)
    # by size on a named group setting: 50 / 50 of the element count
    hcom.set_grad_fusion_by_size("odd", [50.0, 50.0])
    cuts = grad_bucket.plan_segments([10, 10, 10, 10], group="odd")
    assert cuts == [(0, 2), (2, 4)], cuts
    td = c.topo_desc()
    assert td[0][1] == p and td[0][0] & L.ALG_MESH and td[1] == (0, 0)
    hcom.destroy_group("odd")
    hcom.destroy()
    x = np.ones(8, np.float32)
    out = np.zeros_like(x)
    c.all_reduce(x, out)        # the adopted world communicator outlives the front end
    np.testing.assert_array_equal(out, np.full(8, p, np.float32))
    print("hcom ok")


def scenario_onesided(c, p, r, args):
    """Put / get on symmetric memory, topology JSON, overflow counter."""
    n = 256
    handle, (buf,) = c.symmetric_empty(n * p, np.float32)
    buf[:] = -1
    c.barrier()
    mine = np.full(n, r + 1, np.float32)
    for q in range(p):      # everyone writes its block into slot r of every rank's copy
        c.put(handle, q, r * n * 4, mine.ctypes.data, n * 4)
    c.barrier()
    np.testing.assert_array_equal(buf.reshape(p, n), np.repeat(np.arange(1, p + 1, dtype=np.float32)[:, None], n, 1))
    got = np.zeros(n, np.float32)
    c.get(handle, (r + 1) % p, ((r + 1) % p) * n * 4, got.ctypes.data, n * 4)
    np.testing.assert_array_equal(got, np.full(n, (r + 1) % p + 1, np.float32))
    try:
        c.put(handle, 0, n * p * 4 - 8, mine.ctypes.data, 64)
        raise AssertionError("out-of-range put accepted")
    except H.HcclError as e:
        assert e.code == L.E_PARA
    c.barrier()
    del buf
    c.mem_free(handle)
    topo = c.topology()
    assert topo["ranks"] == p and topo["transport"] == "host" and len(topo["rank_table"]) == p
    assert [e["rank"] for e in topo["rank_table"]] == list(range(p)) and topo["rank_table"][r]["pid"] == os.getpid()
    # overflow: rank 0 contributes an Inf to the second AllReduce only
    assert c.overflow_count() == 0
    x = np.ones(32, np.float32)
    out = np.zeros_like(x)
    c.all_reduce(x, out)
    assert c.overflow_count() == 0
    if r == 0:
        x[3] = np.inf
    c.all_reduce(x, out)
    assert c.overflow_count() == 1, c.overflow_count()
    print("onesided ok")


def scenario_mismatch(c, p, r, args):
    """rank 1 passes a different count: the consistency check must fail the call on every rank."""
    n = 100 if r != 1 else 101
    x = np.zeros(n, np.float32)
    try:
        c.all_reduce(x, x.copy())
    except H.HcclError as e:
        assert e.code == L.E_PARA, e
        print("mismatch detected")
        return
    raise AssertionError("mismatch not detected")


def scenario_timeout_absent_peer(c, p, r, args):
    """rank 1 never calls the collective: the others' bounded waits must end with HCCL_E_TIMEOUT and a status block."""
    if r == 1:
        time.sleep(float(args[0]))
        print("rank 1 skipped the op")
        return
    x = np.ones(1000, np.float32)
    t0 = time.time()
    try:
        c.all_reduce(x, x.copy(), algo=L.ALGO_MESH)
    except H.HcclError as e:
        assert e.code in (L.E_TIMEOUT, L.E_REMOTE), e
        st = c.status()
        assert st.code == e.code and (st.peer == 1 or e.code == L.E_REMOTE)
        print("timeout after %.2fs: %s" % (time.time() - t0, c.describe_status()))
        assert c.async_error() == e.code
        # the communicator refuses further work until it is resumed
        try:
            c.all_reduce(x, x.copy())
            raise AssertionError("op accepted after failure")
        except H.HcclError as e2:
            assert e2.code == e.code
        return
    raise AssertionError("no timeout")


def scenario_retry(c, p, r, args):
    """HCCL_FAULT_INJECT stalls rank 1 beyond the exec timeout on its 2nd op; with retry enabled all ranks agree to
    re-run it and the result is correct."""
    for i in range(3):
        x = np.full(5000, r + i, np.float32)
        out = np.zeros_like(x)
        c.all_reduce(x, out, algo=L.ALGO_MESH)
        np.testing.assert_array_equal(out, np.full(5000, sum(q + i for q in range(p)), np.float32))
    st = c.stats()
    print("retries:", st["retries"], "timeouts:", st["timeouts"])
    assert st["retries"] >= 1


def scenario_peer_exit(c, p, r, args):
    """rank 2 exits before its 2nd op (fault injection).  Survivors learn it from the heartbeat (rank lost) or from
    their bounded wait, and HcclGetCommAsyncError reports it."""
    x = np.ones(100, np.float32)
    c.all_reduce(x, x.copy())
    t0 = time.time()
    try:
        c.all_reduce(x, x.copy())
    except H.HcclError as e:
        assert e.code in (L.E_TIMEOUT, L.E_REMOTE), e
        print("peer loss seen after %.2fs as %d; async error %d" % (time.time() - t0, e.code, c.async_error()))
        assert c.async_error() != 0
        os._exit(0)  # peers are gone: skip the collective teardown
    raise AssertionError("peer exit not noticed")


def scenario_suspend_resume(c, p, r, args):
    x = np.ones(64, np.float32)
    c.all_reduce(x, x.copy())
    c.suspend()
    try:
        c.all_reduce(x, x.copy())
        raise AssertionError("suspended communicator accepted an op")
    except H.HcclError as e:
        assert e.code == L.E_SUSPENDING
    c.resume()
    out = np.zeros_like(x)
    c.all_reduce(x, out)
    np.testing.assert_array_equal(out, np.full(64, p, np.float32))
    print("suspend/resume ok")


def scenario_staged_abort(c, p, r, args):
    """The three abort stages with time budgets (HcclB200TaskAbort).  Rank 1 enters its 2nd collective late (host-side
    stall of 3 s inside the call), so rank 0 sits in a bounded wait: stage 0 tells both to stop.  On rank 1 the stalled
    call cannot leave within a 1 s budget (result 2 = timed out); asked again without limit it succeeds."""
    import threading
    lib = L.lib()
    lib.HcclB200TaskAbort.restype = C.c_int32
    lib.HcclB200TaskAbort.argtypes = [C.c_int32, C.c_int32, C.c_uint32]
    x = np.ones(64, np.float32)
    c.all_reduce(x, x.copy())
    res = {}

    def op():
        try:
            c.all_reduce(x, x.copy())
            res["rc"] = 0
        except H.HcclError as e:
            res["rc"] = e.code
    t = threading.Thread(target=op)
    t.start()
    time.sleep(0.5)                                  # both ranks are inside the call now (rank 1 in its stall)
    first = lib.HcclB200TaskAbort(-1, 0, 1)
    if r == 1:
        assert first == 2, first                     # the stalled call holds the communicator beyond the budget
        assert lib.HcclB200TaskAbort(-1, 0, 0) == 0  # no limit: returns once the call has left
    else:
        assert first == 0, first
    t.join()
    assert res["rc"] == L.E_SUSPENDING, res
    assert lib.HcclB200TaskAbort(-1, 1, 5) == 0
    assert lib.HcclB200TaskAbort(-1, 2, 5) == 0
    assert c.status().code == 0
    c.resume()
    out = np.zeros_like(x)
    c.all_reduce(x, out)
    np.testing.assert_array_equal(out, np.full(64, p, np.float32))
    print("staged abort ok")


def scenario_stuck(c, p, r, args):
    """rank 1 stalls inside... before its op for longer than HCCL_STUCK_DETECT_MS while rank 0 waits in the op:
    rank 0's heartbeat thread reports itself stuck; rank 1 (idle, healthy) learns of it through the hub."""
    x = np.ones(16, np.float32)
    if r == 1:
        t0 = time.time()
        while time.time() - t0 < 6 and c.async_error() == 0:
            time.sleep(0.05)
        assert c.async_error() == L.E_TIMEOUT, c.async_error()
        print("stuck peer reported")
        os._exit(0)
    try:
        c.all_reduce(x, x.copy())
    except H.HcclError:
        pass
    os._exit(0)


if __name__ == "__main__":
    scenario, p, r, root_file = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    comm = make_comm(p, r, root_file)
    globals()["scenario_" + scenario](comm, p, r, sys.argv[5:])
    code = comm.destroy()
    assert code == L.SUCCESS, code
