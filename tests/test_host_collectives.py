"""Every collective x algorithm x rank count on the host-memory transport against the numpy oracle.

The same plans run on the GPU executor; what is checked here is the schedule logic (slices, dependencies,
fold/unfold for non-power-of-two ranks, staging loop), which needs no GPU.
"""
import numpy as np
import pytest

import cann_hccl_b200 as H
from cann_hccl_b200 import _lib as L
from oracle import make_inputs, np_reduce, tol

RANKS = [2, 3, 4, 5, 7, 8]


@pytest.fixture(scope="module")
def comms():
    cache = {}

    def get(p):
        if p not in cache:
            cfg = L.CommConfig.default()
            cfg.hcclBufferSize = 1  # 1 MB staging halves: larger messages exercise the staging loop
            cache[p] = H.Communicator.init_local(p, device=False, config=cfg)
        return cache[p]

    yield get
    for c in cache.values():
        assert c.destroy() == L.SUCCESS


@pytest.mark.parametrize("p", RANKS)
@pytest.mark.parametrize("algo", [L.ALGO_MESH_ONESHOT, L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD])
@pytest.mark.parametrize("n", [1, 7, 1000, 4099])
def test_allreduce_algos(comms, p, algo, n):
    c = comms(p)
    ins = make_inputs(p, n, np.float32)
    outs = [np.zeros(n, np.float32) for _ in range(p)]
    c.all_reduce(ins, outs, algo=algo, nchan=3)
    ref = np_reduce(ins, L.SUM)
    for o in outs:
        np.testing.assert_allclose(o, ref, **tol(np.float32, p))


@pytest.mark.parametrize("dtype", [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64,
                                   np.float16, np.float32, np.float64])
@pytest.mark.parametrize("op", [L.SUM, L.PROD, L.MAX, L.MIN])
def test_allreduce_dtypes_ops(comms, dtype, op):
    p, n = 4, 257
    c = comms(p)
    ins = make_inputs(p, n, dtype)
    outs = [np.zeros(n, dtype) for _ in range(p)]
    c.all_reduce(ins, outs, op=op, algo=L.ALGO_MESH)
    ref = np_reduce(ins, op)
    for o in outs:
        np.testing.assert_allclose(o.astype(np.float64), ref.astype(np.float64), **tol(dtype, p))


@pytest.mark.parametrize("p", [2, 3])
def test_pipelined_algorithms_fall_back_on_cpu_ranks(comms, p):
    """The pipelined kernels exist on the device only; CPU ranks asked for them run the plain schedule of the same family."""
    c = comms(p)
    n = 20_003
    ins = make_inputs(p, n, np.float32)
    outs = [np.zeros(n, np.float32) for _ in range(p)]
    c.all_reduce(ins, outs, algo=L.ALGO_MESH_PIPE)
    ref = np_reduce(ins, L.SUM)
    for o in outs:
        np.testing.assert_allclose(o, ref, **tol(np.float32, p))
    bufs = make_inputs(p, n, np.float32)
    want = bufs[1].copy()
    c.broadcast(bufs, 1, algo=L.ALGO_MESH_PIPE)
    for b in bufs:
        np.testing.assert_array_equal(b, want)


def test_buffer_overlap_rules(comms):
    """In place means one of the forms the op defines (same pointer; own block at its position of the larger buffer).
    Buffers that overlap in any other way are refused before anything runs, whatever the algorithm."""
    p, n = 4, 1000
    c = comms(p)
    base = [np.arange(2 * n * p, dtype=np.float32) + r for r in range(p)]
    # AllReduce: shifted by one element -> refused; equal pointers -> fine
    with pytest.raises(H.HcclError) as e:
        c.all_reduce([b[:n] for b in base], [b[1:n + 1] for b in base])
    assert e.value.code == L.E_PARA
    ins = [b[:n].copy() for b in base]
    ref = np_reduce(ins, L.SUM)
    views = [b[:n] for b in base]
    c.all_reduce(views, views)
    for v in views:
        np.testing.assert_allclose(v, ref, **tol(np.float32, p))
    # AllGather: the send buffer inside the receive buffer but not at the rank's own block -> refused
    full = [np.zeros(n * p, np.float32) for _ in range(p)]
    with pytest.raises(H.HcclError) as e:
        c.all_gather([f[:n] for f in full], full)          # every rank offers block 0: only right for rank 0
    assert e.value.code == L.E_PARA
    gs = make_inputs(p, n, np.float32)
    for r in range(p):
        full[r][r * n:(r + 1) * n] = gs[r]
    c.all_gather([full[r][r * n:(r + 1) * n] for r in range(p)], full)
    for f in full:
        np.testing.assert_array_equal(f, np.concatenate(gs))
    # ReduceScatter: receive buffer = the rank's own block of the send buffer is in place; any other block is refused
    xs = make_inputs(p, n * p, np.float32)
    want = np_reduce(xs, L.SUM)
    work = [x.copy() for x in xs]
    with pytest.raises(H.HcclError) as e:
        c.reduce_scatter(work, [w[n // 2:n // 2 + n] for w in work])
    assert e.value.code == L.E_PARA
    c.reduce_scatter(work, [work[r][r * n:(r + 1) * n] for r in range(p)])
    for r in range(p):
        np.testing.assert_allclose(work[r][r * n:(r + 1) * n], want[r * n:(r + 1) * n], **tol(np.float32, p))


def test_allreduce_bf16_bits(comms):
    """bf16 travels as uint16 through numpy; the library reduces it in fp32 and rounds once."""
    import ctypes as C
    p, n = 4, 300
    c = comms(p)
    rng = np.random.default_rng(0)
    f = [rng.uniform(-1, 1, n).astype(np.float32) for _ in range(p)]
    bf = [(x.view(np.uint32) >> 16).astype(np.uint16) for x in f]  # truncation gives exact bf16 values
    exact = [(b.astype(np.uint32) << 16).view(np.float32) for b in bf]
    outs = [np.zeros(n, np.uint16) for _ in range(p)]
    o = L.B200Op()
    o.coll, o.algo, o.dataType, o.op, o.count = L.ALLREDUCE, L.ALGO_MESH, L.BFP16, L.SUM, n
    sa = (C.c_void_p * p)(*[b.ctypes.data for b in bf])
    ra = (C.c_void_p * p)(*[b.ctypes.data for b in outs])
    L.check(L.lib().HcclB200Collective(c.handle, C.byref(o), sa, ra, None), "bf16 allreduce")
    ref = sum(exact)
    for out in outs:
        got = (out.astype(np.uint32) << 16).view(np.float32)
        np.testing.assert_allclose(got, ref, rtol=1e-2, atol=2e-2)


def test_allreduce_in_place_and_staging_loop(comms):
    p, n = 4, 700_000  # 2.8 MB per rank through 1 MB staging halves -> several loop iterations
    c = comms(p)
    for algo in [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD, L.ALGO_MESH_ONESHOT]:
        ins = make_inputs(p, n, np.float32)
        ref = np_reduce(ins, L.SUM)
        c.all_reduce(ins, ins, algo=algo, nchan=2)
        for o in ins:
            np.testing.assert_allclose(o, ref, **tol(np.float32, p))
    assert c.stats()["launches"] > 8


@pytest.mark.parametrize("p", RANKS)
@pytest.mark.parametrize("algo", [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD])
@pytest.mark.parametrize("n", [1, 33, 1025])
def test_reduce_scatter(comms, p, algo, n):
    c = comms(p)
    ins = make_inputs(p, n * p, np.float32)
    outs = [np.zeros(n, np.float32) for _ in range(p)]
    c.reduce_scatter(ins, outs, algo=algo, nchan=2)
    ref = np_reduce(ins, L.SUM)
    for r, o in enumerate(outs):
        np.testing.assert_allclose(o, ref[r * n:(r + 1) * n], **tol(np.float32, p))


@pytest.mark.parametrize("p", RANKS)
@pytest.mark.parametrize("algo", [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD, L.ALGO_PAIRWISE])
@pytest.mark.parametrize("n", [1, 33, 1025])
def test_all_gather(comms, p, algo, n):
    c = comms(p)
    ins = make_inputs(p, n, np.int32)
    outs = [np.zeros(n * p, np.int32) for _ in range(p)]
    c.all_gather(ins, outs, algo=algo, nchan=2)
    ref = np.concatenate(ins)
    for o in outs:
        np.testing.assert_array_equal(o, ref)


def test_all_gather_in_place_large(comms):
    p, n = 4, 300_000
    c = comms(p)
    for algo in [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD, L.ALGO_PAIRWISE]:
        ins = make_inputs(p, n, np.float32)
        outs = [np.zeros(n * p, np.float32) for _ in range(p)]
        for r in range(p):
            outs[r][r * n:(r + 1) * n] = ins[r]
        views = [outs[r][r * n:(r + 1) * n] for r in range(p)]
        c.all_gather(views, outs, algo=algo)
        ref = np.concatenate(ins)
        for o in outs:
            np.testing.assert_array_equal(o, ref)


@pytest.mark.parametrize("p", [2, 3, 4, 8])
@pytest.mark.parametrize("algo", [L.ALGO_MESH, L.ALGO_RING])
def test_v_variants(comms, p, algo):
    c = comms(p)
    rng = np.random.default_rng(5)
    counts = rng.integers(0, 50, p).astype(np.uint64)
    counts[0] = 17
    displs = np.zeros(p, np.uint64)
    gap = 3
    for j in range(1, p):
        displs[j] = displs[j - 1] + counts[j - 1] + gap
    total = int(displs[-1] + counts[-1])
    # AllGatherV
    ins = [rng.standard_normal(int(counts[r])).astype(np.float32) for r in range(p)]
    outs = [np.full(total, -7, np.float32) for _ in range(p)]
    c.all_gather_v(ins, outs, counts, displs, algo=algo)
    for o in outs:
        for j in range(p):
            np.testing.assert_array_equal(o[int(displs[j]):int(displs[j] + counts[j])], ins[j])
    if algo == L.ALGO_MESH:  # the push variant exists for the gather side only
        outs = [np.full(total, -7, np.float32) for _ in range(p)]
        c.all_gather_v(ins, outs, counts, displs, algo=L.ALGO_PAIRWISE)
        for o in outs:
            for j in range(p):
                np.testing.assert_array_equal(o[int(displs[j]):int(displs[j] + counts[j])], ins[j])
    # ReduceScatterV
    ins = [rng.standard_normal(total).astype(np.float32) for _ in range(p)]
    outs = [np.zeros(max(1, int(counts[r])), np.float32) for r in range(p)]
    c.reduce_scatter_v(ins, outs, counts, displs, algo=algo)
    ref = np_reduce(ins, L.SUM)
    for r in range(p):
        np.testing.assert_allclose(outs[r][:int(counts[r])], ref[int(displs[r]):int(displs[r] + counts[r])], **tol(np.float32, p))


@pytest.mark.parametrize("p", RANKS)
@pytest.mark.parametrize("algo", [L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE])
def test_broadcast(comms, p, algo):
    c = comms(p)
    for root in {0, p - 1, p // 2}:
        n = 1234
        bufs = make_inputs(p, n, np.float32, seed=root)
        ref = bufs[root].copy()
        c.broadcast(bufs, root, algo=algo, nchan=2)
        for b in bufs:
            np.testing.assert_array_equal(b, ref)


@pytest.mark.parametrize("p", RANKS)
@pytest.mark.parametrize("algo", [L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE, L.ALGO_RHD])
def test_reduce(comms, p, algo):
    c = comms(p)
    for root in {0, p - 1}:
        n = 999
        ins = make_inputs(p, n, np.float32)
        outs = [np.full(n, 5, np.float32) for _ in range(p)]
        c.reduce(ins, outs, root, algo=algo, nchan=2)
        np.testing.assert_allclose(outs[root], np_reduce(ins, L.SUM), **tol(np.float32, p))


@pytest.mark.parametrize("p", RANKS)
@pytest.mark.parametrize("algo", [L.ALGO_STAR, L.ALGO_RING])
def test_scatter_gather(comms, p, algo):
    c = comms(p)
    n = 321
    for root in {0, p - 1}:
        ins = make_inputs(p, n * p, np.int32)
        outs = [np.zeros(n, np.int32) for _ in range(p)]
        c.scatter(ins, outs, root, algo=algo, nchan=2)
        for r in range(p):
            np.testing.assert_array_equal(outs[r], ins[root][r * n:(r + 1) * n])
        gin = make_inputs(p, n, np.int32, seed=77)
        gout = [np.zeros(n * p, np.int32) for _ in range(p)]
        c.gather(gin, gout, root, algo=algo, nchan=2)
        np.testing.assert_array_equal(gout[root], np.concatenate(gin))


@pytest.mark.parametrize("p", RANKS)
@pytest.mark.parametrize("algo", [L.ALGO_MESH, L.ALGO_PAIRWISE])
def test_all_to_all(comms, p, algo):
    c = comms(p)
    n = 77
    ins = make_inputs(p, n * p, np.float32)
    outs = [np.zeros(n * p, np.float32) for _ in range(p)]
    c.all_to_all(ins, outs, algo=algo, nchan=2)
    for r in range(p):
        for q in range(p):
            np.testing.assert_array_equal(outs[r][q * n:(q + 1) * n], ins[q][r * n:(r + 1) * n])


@pytest.mark.parametrize("p", [2, 3, 4, 8])
@pytest.mark.parametrize("algo", [L.ALGO_MESH, L.ALGO_PAIRWISE])
@pytest.mark.parametrize("scale", [40, 60000])
def test_all_to_all_v(comms, p, algo, scale):
    """Uneven counts; `scale`=60000 makes blocks exceed a staging slot (1 MB / p), so rounds with acks run."""
    c = comms(p)
    rng = np.random.default_rng(7)
    m = rng.integers(0, scale, (p, p)).astype(np.uint64)  # m[i][j]: elements rank i sends to rank j
    m[0, 1] = 0
    sd = np.zeros((p, p), np.uint64)
    rd = np.zeros((p, p), np.uint64)
    for i in range(p):
        sd[i] = np.concatenate([[0], np.cumsum(m[i])[:-1]])
        rd[i] = np.concatenate([[0], np.cumsum(m[:, i])[:-1]])
    ins = [rng.standard_normal(int(m[i].sum()) + 1).astype(np.float32) for i in range(p)]
    outs = [np.zeros(int(m[:, i].sum()) + 1, np.float32) for i in range(p)]
    rc = np.ascontiguousarray(m.T)
    c.all_to_all_v(ins, m, sd, outs, rc, rd, algo=algo, nchan=2)
    for i in range(p):
        for j in range(p):
            got = outs[j][int(rd[j, i]):int(rd[j, i] + m[i, j])]
            want = ins[i][int(sd[i, j]):int(sd[i, j] + m[i, j])]
            np.testing.assert_array_equal(got, want)


def test_all_to_all_v_count_matrix_mismatch_is_refused(comms):
    """What rank i sends to j must be what j expects from i; a matrix that disagrees is refused before any data moves."""
    p = 3
    c = comms(p)
    m = np.full((p, p), 5, np.uint64)
    rc = np.ascontiguousarray(m.T)
    rc[2, 0] = 6                                        # rank 2 expects 6 elements from rank 0, which sends 5
    sd = np.tile(np.arange(p, dtype=np.uint64) * 5, (p, 1))
    rd = np.tile(np.arange(p, dtype=np.uint64) * 6, (p, 1))
    ins = [np.zeros(32, np.float32) for _ in range(p)]
    outs = [np.zeros(32, np.float32) for _ in range(p)]
    with pytest.raises(H.HcclError) as e:
        c.all_to_all_v(ins, m, sd, outs, rc, rd)
    assert e.value.code == L.E_PARA


def test_barrier_and_single_rank(comms):
    c = comms(4)
    c.barrier()
    one = H.Communicator.init_local(1, device=False)
    a = np.arange(10, dtype=np.float32)
    b = np.zeros(10, np.float32)
    one.all_reduce([a], [b])
    np.testing.assert_array_equal(a, b)
    one.all_gather([a], [b])
    np.testing.assert_array_equal(a, b)
    one.barrier()
    assert one.destroy() == L.SUCCESS


def test_local_send_recv(comms):
    c = comms(4)
    for n in [5, 100_000]:  # 400 KB > one 256 KB mailbox slot -> two rounds with an acknowledgement
        a = np.arange(n, dtype=np.float32)
        b = np.zeros(n, np.float32)
        c.local_send_recv(1, 3, a, b)
        np.testing.assert_array_equal(a, b)
        c.local_send_recv(3, 1, b, a)
    c.local_send_recv(1, 3, a, b)
    np.testing.assert_array_equal(a, b)


def test_auto_selection_runs(comms):
    c = comms(8)
    for n in [16, 5000, 200_000]:
        ins = make_inputs(8, n, np.float32)
        outs = [np.zeros(n, np.float32) for _ in range(8)]
        c.all_reduce(ins, outs)
        np.testing.assert_allclose(outs[3], np_reduce(ins, L.SUM), **tol(np.float32, 8))
    tr = c.trace()
    assert tr and tr[-1]["op"] == "AllReduce" and tr[-1]["algo"] in L.ALGO_NAMES


@pytest.mark.parametrize("p", [2, 5, 8])
def test_zero_copy_allreduce_on_registered_memory(comms, p):
    """Buffers in registered symmetric memory: the zero-copy plan reduces straight from the send buffers into the receive
    buffers of every rank (host executor emulates the multicast accesses)."""
    c = comms(p)
    n = 300_000  # 1.2 MB: above the zero-copy threshold
    hin, ins = c.symmetric_empty(n, np.float32)
    hout, outs = c.symmetric_empty(n, np.float32)
    src = make_inputs(p, n, np.float32)
    for r in range(p):
        ins[r][:] = src[r]
        outs[r][:] = 0
    c.all_reduce(ins, outs)
    assert c.trace()[-1]["algo"] == "nvls_zerocopy"
    ref = np_reduce(src, L.SUM)
    for o in outs:
        np.testing.assert_allclose(o, ref, **tol(np.float32, p))
    c.all_reduce(ins, ins)  # in place
    for o in ins:
        np.testing.assert_allclose(o, ref, **tol(np.float32, p))
    del ins, outs
    c.mem_free(hin)
    c.mem_free(hout)


def test_zero_copy_allreduce_on_adopted_user_memory(comms):
    """Caller-owned buffers registered with mem_adopt behave like library-allocated symmetric memory: the zero-copy plan
    runs on them, and mem_free ends the registration without touching the buffers."""
    p = 4
    c = comms(p)
    n = 300_000
    src = make_inputs(p, n, np.float32)
    ins = [s_.copy() for s_ in src]
    outs = [np.zeros(n, np.float32) for _ in range(p)]
    hin, hout = c.mem_adopt(ins), c.mem_adopt(outs)
    c.all_reduce(ins, outs)
    assert c.trace()[-1]["algo"] == "nvls_zerocopy"
    ref = np_reduce(src, L.SUM)
    for o in outs:
        np.testing.assert_allclose(o, ref, **tol(np.float32, p))
    c.mem_free(hin)
    c.mem_free(hout)
    outs2 = [np.zeros(n, np.float32) for _ in range(p)]
    c.all_reduce(ins, outs2)  # registration gone: staged path, same values
    assert c.trace()[-1]["algo"] != "nvls_zerocopy"
    for o in outs2:
        np.testing.assert_allclose(o, ref, **tol(np.float32, p))
    for a, b in zip(ins, src):
        np.testing.assert_array_equal(a, b)
