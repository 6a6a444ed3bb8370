"""GPU executor kernel: every collective and algorithm with virtual ranks on one GPU (one cooperative launch runs all
ranks, peers are other regions of the same device), against a plain PyTorch fp32 reference of the same op."""
import pytest

torch = pytest.importorskip("torch")
import cann_hccl_b200 as H  # noqa: E402
from cann_hccl_b200 import _lib as L  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def comms():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    cache = {}

    def get(p):
        if p not in cache:
            cfg = L.CommConfig.default()
            cfg.hcclBufferSize = 4
            cache[p] = H.Communicator.init_local(p, device=True, device_id=0, config=cfg)
        return cache[p]

    yield get
    for c in cache.values():
        assert c.destroy() == L.SUCCESS


def ok(c):
    rc = c.sync()
    assert rc == 0, c.describe_status()


def ref_reduce(ins, op):
    acc = ins[0].float() if ins[0].dtype in (torch.float16, torch.bfloat16) else ins[0].clone()
    for x in ins[1:]:
        y = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
        acc = {L.SUM: acc + y, L.PROD: acc * y, L.MAX: torch.maximum(acc, y), L.MIN: torch.minimum(acc, y)}[op]
    return acc.to(ins[0].dtype)


def rnd(p, n, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return [(torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype) for _ in range(p)]
    return [torch.randint(-3, 4, (n,), device="cuda", generator=g).to(dtype) for _ in range(p)]


def close(a, b, dtype, p):
    if dtype == torch.float32:
        torch.testing.assert_close(a, b, rtol=1e-6 * p, atol=1e-6 * p)
    elif dtype in (torch.float16, torch.bfloat16):
        torch.testing.assert_close(a.float(), b.float(), rtol=1.6e-2, atol=1.6e-2 * p)
    else:
        assert torch.equal(a, b)


@pytest.mark.parametrize("p", [2, 3, 4, 8])
@pytest.mark.parametrize("algo", [L.ALGO_MESH_ONESHOT, L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD])
@pytest.mark.parametrize("n", [1, 1000, 262147])
def test_allreduce(comms, p, algo, n):
    c = comms(p)
    ins = rnd(p, n, torch.float32)
    outs = [torch.zeros(n, device="cuda") for _ in range(p)]
    c.all_reduce(ins, outs, algo=algo)
    ok(c)
    ref = ref_reduce(ins, L.SUM)
    for o in outs:
        close(o, ref, torch.float32, p)


@pytest.mark.parametrize("dtype", [torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64, torch.float16, torch.bfloat16,
                                   torch.float32, torch.float64])
@pytest.mark.parametrize("op", [L.SUM, L.PROD, L.MAX, L.MIN])
def test_allreduce_dtypes_ops(comms, dtype, op):
    p, n = 4, 4099
    c = comms(p)
    if dtype == torch.uint8:
        ins = [torch.randint(0, 3, (n,), device="cuda", dtype=torch.uint8) for _ in range(p)]
    else:
        ins = rnd(p, n, dtype, seed=3)
    outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(p)]
    c.all_reduce(ins, outs, op=op, algo=L.ALGO_MESH)
    ok(c)
    ref = ref_reduce(ins, op)
    for o in outs:
        close(o, ref, dtype, p)


@pytest.mark.parametrize("p", [2, 3, 8])
@pytest.mark.parametrize("dtype,op", [(torch.float32, L.SUM), (torch.bfloat16, L.SUM), (torch.float16, L.MAX), (torch.int8, L.MIN),
                                      (torch.int64, L.PROD), (torch.float64, L.SUM)])
def test_allreduce_low_latency_protocol(comms, p, dtype, op):
    """LL kernel: data and tag in the same 16-byte line, double-buffered mailboxes; repeated calls alternate parity."""
    c = comms(p)
    for n in (1, 2, 1023, 30001):
        ins = rnd(p, n, dtype, seed=n)
        outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(p)]
        for _ in range(3):
            c.all_reduce(ins, outs, op=op, algo=L.ALGO_LL)
        ok(c)
        ref = ref_reduce(ins, op)
        for o in outs:
            close(o, ref, dtype, p)
    assert c.stats()["algos"].get("ll", 0) >= 12


@pytest.mark.parametrize("p", [2, 4])
def test_allreduce_low_latency_element_aligned_views(comms, p):
    """Views that are only element-aligned on SOME ranks: every rank still runs the LL kernels (which path a rank's loads and
    stores take is its own business), so the ranks cannot end up in different algorithms."""
    c = comms(p)
    for dtype, n in ((torch.float32, 10_001), (torch.bfloat16, 33_333), (torch.float32, 150_000)):  # one-shot; one-shot; two-shot on four ranks
        base_in = rnd(p, n + 3, dtype, seed=n % 53)
        base_out = [torch.zeros(n + 3, device="cuda", dtype=dtype) for _ in range(p)]
        ins = [base_in[r][(r % 2):(r % 2) + n] for r in range(p)]          # odd ranks start one element in
        outs = [base_out[r][((r + 1) % 2) * 3:((r + 1) % 2) * 3 + n] for r in range(p)]  # even ranks' outputs start three elements in
        for _ in range(2):
            c.all_reduce(ins, outs, algo=L.ALGO_LL)
        ok(c)
        assert c.trace()[-1]["algo"] == "ll"
        ref = ref_reduce(ins, L.SUM)
        for o in outs:
            close(o, ref, dtype, p)


@pytest.mark.parametrize("p", [3, 4, 8])
@pytest.mark.parametrize("dtype,op", [(torch.float32, L.SUM), (torch.bfloat16, L.MAX), (torch.int32, L.MIN), (torch.float64, L.PROD)])
def test_allreduce_low_latency_two_shot(comms, p, dtype, op):
    """From 256 KiB on, three and more ranks run the LL protocol two-shot: slices to their owners, reduced slices back."""
    c = comms(p)
    for n in (70_001, 262_144, (p << 20) // dtype.itemsize):   # odd tail; even; the largest message the mailboxes take
        if n * dtype.itemsize < (256 << 10):
            n = (300 << 10) // dtype.itemsize + 3
        ins = rnd(p, n, dtype, seed=n % 61)
        outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(p)]
        for _ in range(3):  # repeated calls alternate the mailbox parity
            c.all_reduce(ins, outs, op=op, algo=L.ALGO_LL)
        ok(c)
        assert c.trace()[-1]["algo"] == "ll"
        ref = ref_reduce(ins, op)
        for o in outs:
            close(o, ref, dtype, p)


@pytest.mark.parametrize("p", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype,op", [(torch.float32, L.SUM), (torch.bfloat16, L.MAX), (torch.int32, L.MIN), (torch.float64, L.PROD)])
def test_reduce_scatter_and_allgather_low_latency(comms, p, dtype, op):
    """The two halves of the two-shot LL AllReduce as collectives of their own; odd counts put the blocks at element-aligned
    addresses only."""
    c = comms(p)
    for n in (1, 1_001, 65_537, (1 << 20) // dtype.itemsize):   # per-rank block; the last is the largest the mailboxes take
        ins = rnd(p, n * p, dtype, seed=n % 59)
        outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(p)]
        for _ in range(3):  # repeated calls alternate the mailbox parity
            c.reduce_scatter(ins, outs, op=op, algo=L.ALGO_LL)
        ok(c)
        assert c.trace()[-1]["algo"] == "ll"
        ref = ref_reduce(ins, op)
        for r, o in enumerate(outs):
            close(o, ref[r * n:(r + 1) * n], dtype, p)
        gs = rnd(p, n, dtype, seed=n % 47)
        gout = [torch.zeros(n * p, device="cuda", dtype=dtype) for _ in range(p)]
        for _ in range(2):
            c.all_gather(gs, gout, algo=L.ALGO_LL)
        ok(c)
        assert c.trace()[-1]["algo"] == "ll"
        for o in gout:
            assert torch.equal(o, torch.cat(gs))
    # in place: AllGather with every rank's block already at its position, ReduceScatter onto the rank's own block
    n = 30_001
    full = [torch.zeros(n * p, device="cuda") for _ in range(p)]
    gs = rnd(p, n, torch.float32, seed=2)
    for r in range(p):
        full[r][r * n:(r + 1) * n] = gs[r]
    c.all_gather([full[r][r * n:(r + 1) * n] for r in range(p)], full, algo=L.ALGO_LL)
    ok(c)
    for o in full:
        assert torch.equal(o, torch.cat(gs))
    ins = rnd(p, n * p, torch.float32, seed=3)
    ref = ref_reduce(ins, L.SUM)
    c.reduce_scatter(ins, [ins[r][r * n:(r + 1) * n] for r in range(p)], algo=L.ALGO_LL)
    ok(c)
    for r in range(p):
        close(ins[r][r * n:(r + 1) * n], ref[r * n:(r + 1) * n], torch.float32, p)
    # one block too large for the mailboxes: the plan executor takes over
    n = (1 << 20) // 4 + 64
    ins = rnd(p, n * p, torch.float32, seed=4)
    outs = [torch.zeros(n, device="cuda") for _ in range(p)]
    c.reduce_scatter(ins, outs, algo=L.ALGO_LL)
    ok(c)
    assert c.trace()[-1]["algo"] == "mesh"
    ref = ref_reduce(ins, L.SUM)
    for r, o in enumerate(outs):
        close(o, ref[r * n:(r + 1) * n], torch.float32, p)


PIPE_SIZES = (5, 70_001, 3_000_000)  # part of a chunk; one chunk; twelve chunks through a four-slot ring (4 MB staging halves)


@pytest.mark.parametrize("p", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype,op", [(torch.float32, L.SUM), (torch.bfloat16, L.MAX), (torch.int32, L.MIN), (torch.float64, L.PROD)])
def test_pipelined_allreduce(comms, p, dtype, op):
    """Pipelined kernel: copy-in, reduce and copy-out stages of one launch over a ring of staging slots (two ranks: one-shot)."""
    c = comms(p)
    for n in PIPE_SIZES:
        ins = rnd(p, n, dtype, seed=n % 89)
        outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(p)]
        c.all_reduce(ins, outs, op=op, algo=L.ALGO_MESH_PIPE)
        ok(c)
        assert c.trace()[-1]["algo"] == "mesh_pipe"
        ref = ref_reduce(ins, op)
        for o in outs:
            close(o, ref, dtype, p)


def test_pipelined_allreduce_in_place_unaligned_back_to_back(comms):
    p = 4
    c = comms(p)
    n = 2_500_001
    base = rnd(p, n + 1, torch.float32, seed=5)
    ins = [b[1:] for b in base]  # 4-byte aligned only: the scalar paths of the copy and reduce loops
    ref = ref_reduce(ins, L.SUM)
    c.all_reduce(ins, ins, algo=L.ALGO_MESH_PIPE)
    ok(c)
    for o in ins:
        close(o, ref, torch.float32, p)
    # consecutive ops alternate staging halves and reuse the arrival counters
    xs = rnd(p, 1_200_000, torch.float32, seed=6)
    outs = [torch.zeros_like(x) for x in xs]
    for _ in range(5):
        c.all_reduce(xs, outs, algo=L.ALGO_MESH_PIPE)
    ok(c)
    for o in outs:
        close(o, ref_reduce(xs, L.SUM), torch.float32, p)


@pytest.mark.parametrize("p", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pipelined_reduce_scatter_allgather(comms, p, dtype):
    c = comms(p)
    for n in (3, 40_001, 700_000):  # per-rank block; the largest runs the ring several times over
        ins = rnd(p, n * p, dtype, seed=n % 83)
        outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(p)]
        c.reduce_scatter(ins, outs, algo=L.ALGO_MESH_PIPE)
        ok(c)
        ref = ref_reduce(ins, L.SUM)
        for r, o in enumerate(outs):
            close(o, ref[r * n:(r + 1) * n], dtype, p)
        gs = rnd(p, n, dtype, seed=n % 79)
        gout = [torch.zeros(n * p, device="cuda", dtype=dtype) for _ in range(p)]
        c.all_gather(gs, gout, algo=L.ALGO_MESH_PIPE)
        ok(c)
        for o in gout:
            assert torch.equal(o, torch.cat(gs))
    # AllGather in place: every rank's block already sits at its position of the receive buffer
    n = 300_001
    full = [torch.zeros(n * p, device="cuda") for _ in range(p)]
    gs = rnd(p, n, torch.float32, seed=2)
    for r in range(p):
        full[r][r * n:(r + 1) * n] = gs[r]
    c.all_gather([full[r][r * n:(r + 1) * n] for r in range(p)], full, algo=L.ALGO_MESH_PIPE)
    ok(c)
    for o in full:
        assert torch.equal(o, torch.cat(gs))


@pytest.mark.parametrize("p", [2, 3, 8])
def test_pipelined_broadcast_chain(comms, p):
    c = comms(p)
    for n, root in ((7, 0), (100_003, p - 1), (2_000_000, 1)):
        bufs = rnd(p, n, torch.float32, seed=n % 71)
        want = bufs[root].clone()
        c.broadcast(bufs, root, algo=L.ALGO_MESH_PIPE)
        ok(c)
        for b in bufs:
            assert torch.equal(b, want)


@pytest.mark.parametrize("p", [2, 3, 4, 8])
@pytest.mark.parametrize("dtype,op", [(torch.float32, L.SUM), (torch.bfloat16, L.MAX)])
def test_pipelined_reduce(comms, p, dtype, op):
    """Reduce as a pipelined two-shot: slices to their owners, reduced slices to the root, which alone copies out."""
    c = comms(p)
    for n, root in ((5, 0), (70_001, p - 1), (3_000_000, 1)):
        ins = rnd(p, n, dtype, seed=n % 67)
        keep = [x.clone() for x in ins]
        outs = [torch.full((n,), 7, device="cuda", dtype=dtype) for _ in range(p)]
        c.reduce(ins, outs, root, op=op, algo=L.ALGO_MESH_PIPE)
        ok(c)
        assert c.trace()[-1]["algo"] == "mesh_pipe"
        close(outs[root], ref_reduce(keep, op), dtype, p)
        for r in range(p):
            assert torch.equal(ins[r], keep[r])
            if r != root:
                assert bool((outs[r] == 7).all())  # only the root's receive buffer is written
    # in place on the root, back to back (the staging halves alternate)
    n = 1_200_000
    ins = rnd(p, n, torch.float32, seed=3)
    ref = ref_reduce(ins, L.SUM)
    for _ in range(3):
        xs = [x.clone() for x in ins]
        c.reduce(xs, xs, 0, algo=L.ALGO_MESH_PIPE)
    ok(c)
    close(xs[0], ref, torch.float32, p)


def test_allreduce_staging_loop_in_place_unaligned(comms):
    p = 4
    c = comms(p)
    n = 3_000_001  # 12 MB through 4 MB staging halves
    for algo in (L.ALGO_MESH, L.ALGO_RING, L.ALGO_MESH_ONESHOT, L.ALGO_RHD):
        base = rnd(p, n + 1, torch.float32, seed=algo)
        ins = [b[1:] for b in base]  # 4-byte aligned only: the scalar path of the kernel
        ref = ref_reduce(ins, L.SUM)
        c.all_reduce(ins, ins, algo=algo)
        ok(c)
        for o in ins:
            close(o, ref, torch.float32, p)


@pytest.mark.parametrize("p", [2, 3, 8])
@pytest.mark.parametrize("algo", [L.ALGO_MESH, L.ALGO_RING, L.ALGO_RHD])
def test_reduce_scatter_all_gather(comms, p, algo):
    c = comms(p)
    n = 5003
    ins = rnd(p, n * p, torch.bfloat16, seed=1)
    outs = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(p)]
    c.reduce_scatter(ins, outs, algo=algo)
    ok(c)
    ref = ref_reduce(ins, L.SUM)
    for r, o in enumerate(outs):
        close(o, ref[r * n:(r + 1) * n], torch.bfloat16, p)
    gins = rnd(p, n, torch.int32, seed=2)
    gouts = [torch.zeros(n * p, device="cuda", dtype=torch.int32) for _ in range(p)]
    c.all_gather(gins, gouts, algo=algo)
    ok(c)
    for o in gouts:
        assert torch.equal(o, torch.cat(gins))
    if algo == L.ALGO_MESH:  # push variant: remote stores into the peers' staging slots
        gouts = [torch.zeros(n * p, device="cuda", dtype=torch.int32) for _ in range(p)]
        c.all_gather(gins, gouts, algo=L.ALGO_PAIRWISE)
        ok(c)
        for o in gouts:
            assert torch.equal(o, torch.cat(gins))


@pytest.mark.parametrize("p", [2, 5, 8])
def test_rooted(comms, p):
    c = comms(p)
    n = 7001
    for root in (0, p - 1):
        for algo in (L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE):
            bufs = rnd(p, n, torch.float32, seed=root)
            ref = bufs[root].clone()
            c.broadcast(bufs, root, algo=algo)
            ok(c)
            for b in bufs:
                assert torch.equal(b, ref)
        for algo in (L.ALGO_STAR, L.ALGO_RING, L.ALGO_TREE, L.ALGO_RHD):
            ins = rnd(p, n, torch.float32, seed=9)
            outs = [torch.zeros(n, device="cuda") for _ in range(p)]
            c.reduce(ins, outs, root, algo=algo)
            ok(c)
            close(outs[root], ref_reduce(ins, L.SUM), torch.float32, p)
        for algo in (L.ALGO_STAR, L.ALGO_RING):
            ins = rnd(p, n * p, torch.int32, seed=4)
            outs = [torch.zeros(n, device="cuda", dtype=torch.int32) for _ in range(p)]
            c.scatter(ins, outs, root, algo=algo)
            ok(c)
            for r in range(p):
                assert torch.equal(outs[r], ins[root][r * n:(r + 1) * n])
            gins = rnd(p, n, torch.int32, seed=5)
            gouts = [torch.zeros(n * p, device="cuda", dtype=torch.int32) for _ in range(p)]
            c.gather(gins, gouts, root, algo=algo)
            ok(c)
            assert torch.equal(gouts[root], torch.cat(gins))


@pytest.mark.parametrize("p", [2, 4, 8])
@pytest.mark.parametrize("algo", [L.ALGO_MESH, L.ALGO_PAIRWISE])
def test_all_to_all_and_v(comms, p, algo):
    import numpy as np
    c = comms(p)
    n = 513
    ins = rnd(p, n * p, torch.float32, seed=6)
    outs = [torch.zeros(n * p, device="cuda") for _ in range(p)]
    c.all_to_all(ins, outs, algo=algo)
    ok(c)
    for r in range(p):
        for q in range(p):
            assert torch.equal(outs[r][q * n:(q + 1) * n], ins[q][r * n:(r + 1) * n])
    rng = np.random.default_rng(7)
    m = rng.integers(0, 300_000 // p, (p, p)).astype(np.uint64)
    sd = np.zeros((p, p), np.uint64)
    rd = np.zeros((p, p), np.uint64)
    for i in range(p):
        sd[i] = np.concatenate([[0], np.cumsum(m[i])[:-1]])
        rd[i] = np.concatenate([[0], np.cumsum(m[:, i])[:-1]])
    vin = [torch.randn(int(m[i].sum()) + 1, device="cuda") for i in range(p)]
    vout = [torch.zeros(int(m[:, i].sum()) + 1, device="cuda") for i in range(p)]
    c.all_to_all_v(vin, m, sd, vout, np.ascontiguousarray(m.T), rd, algo=algo)
    ok(c)
    for i in range(p):
        for j in range(p):
            assert torch.equal(vout[j][int(rd[j, i]):int(rd[j, i] + m[i, j])], vin[i][int(sd[i, j]):int(sd[i, j] + m[i, j])])


@pytest.mark.parametrize("p", [2, 3, 8])
def test_all_to_all_v_parametric_kernel(comms, p):
    """Auto selection on the device runs the parametric kernel: counts travel as launch arguments, so hundreds of distinct
    count matrices build no plan and allocate nothing; blocks larger than a sub-slot go in acknowledged rounds."""
    import numpy as np
    c = comms(p)
    rng = np.random.default_rng(11)
    cap = 200_000 // p
    vin = [torch.randn(cap * p + 8, device="cuda") for _ in range(p)]
    vout = [torch.zeros(cap * p + 8, device="cuda") for _ in range(p)]
    # 4 MB staging halves / (p ranks x lanes x 2) gives sub-slots far below 4 x cap bytes: several rounds per pair
    plans0 = None
    free0 = None
    for it in range(120):
        m = rng.integers(0, cap if it % 7 else 64, (p, p)).astype(np.uint64)
        if it % 5 == 0:
            m[0, p - 1] = 0
        sd = np.zeros((p, p), np.uint64)
        rd = np.zeros((p, p), np.uint64)
        for i in range(p):
            sd[i] = np.concatenate([[0], np.cumsum(m[i])[:-1]])
            rd[i] = np.concatenate([[0], np.cumsum(m[:, i])[:-1]])
        c.all_to_all_v(vin, m, sd, vout, np.ascontiguousarray(m.T), rd)
        if it in (0, 60, 119):
            ok(c)
            assert c.trace()[-1]["algo"] == "direct"
            for i in range(p):
                for j in range(p):
                    assert torch.equal(vout[j][int(rd[j, i]):int(rd[j, i] + m[i, j])], vin[i][int(sd[i, j]):int(sd[i, j] + m[i, j])])
        if it == 0:
            torch.cuda.synchronize()
            plans0, free0 = c.stats()["plans_built"], torch.cuda.mem_get_info()[0]
    ok(c)
    assert c.stats()["plans_built"] == plans0
    assert torch.cuda.mem_get_info()[0] == free0
    # uniform AlltoAll through the same kernel
    n = 70_001
    ins = rnd(p, n * p, torch.float32, seed=8)
    outs = [torch.zeros(n * p, device="cuda") for _ in range(p)]
    c.all_to_all(ins, outs)
    ok(c)
    for r in range(p):
        for q in range(p):
            assert torch.equal(outs[r][q * n:(q + 1) * n], ins[q][r * n:(r + 1) * n])


@pytest.mark.parametrize("p", [2, 4])
def test_zero_copy_over_peer_mappings(comms, p):
    """Send buffers in registered symmetric memory: the peers read them in place (no staging, no chunks).  Two-rank
    AllReduce, ReduceScatter and AllGather; the receive buffers are ordinary tensors."""
    c = comms(p)
    n = 400_003
    hin, zin = c.symmetric_empty(n * p, torch.float32)
    xs = rnd(p, n * p, torch.float32, seed=31)
    for z, x in zip(zin, xs):
        z.copy_(x)
    try:
        outs = [torch.zeros(n, device="cuda") for _ in range(p)]
        for _ in range(2):
            c.reduce_scatter(zin, outs)
        ok(c)
        assert c.trace()[-1]["algo"] == "mesh_zerocopy", c.trace()[-1]
        ref = ref_reduce(xs, L.SUM)
        for r, o in enumerate(outs):
            close(o, ref[r * n:(r + 1) * n], torch.float32, p)
        gout = [torch.zeros(n * p, device="cuda") for _ in range(p)]
        c.all_gather([z[:n] for z in zin], gout)
        ok(c)
        assert c.trace()[-1]["algo"] == "mesh_zerocopy", c.trace()[-1]
        for o in gout:
            assert torch.equal(o, torch.cat([x[:n] for x in xs]))
        if p == 2:
            aouts = [torch.zeros(n * p, device="cuda") for _ in range(p)]
            c.all_reduce(zin, aouts)
            ok(c)
            assert c.trace()[-1]["algo"] == "mesh_zerocopy", c.trace()[-1]
            for o in aouts:
                close(o, ref, torch.float32, p)
            c.all_reduce(zin, zin)   # in place would overwrite what the peer still reads: this form takes a staged path
            ok(c)
            assert c.trace()[-1]["algo"] != "mesh_zerocopy", c.trace()[-1]
            for z in zin:
                close(z, ref, torch.float32, p)
    finally:
        del zin
        c.mem_free(hin)


def test_v_variants_barrier_sendrecv(comms):
    import numpy as np
    p = 4
    c = comms(p)
    counts = np.array([5, 0, 1000, 33], np.uint64)
    displs = np.array([0, 8, 16, 1100], np.uint64)
    total = 1140
    ins = [torch.randn(int(counts[r]), device="cuda") for r in range(p)]
    outs = [torch.full((total,), -1.0, device="cuda") for _ in range(p)]
    c.all_gather_v(ins, outs, counts, displs, algo=L.ALGO_MESH)
    ok(c)
    for o in outs:
        for j in range(p):
            assert torch.equal(o[int(displs[j]):int(displs[j] + counts[j])], ins[j])
    rin = [torch.randn(total, device="cuda") for _ in range(p)]
    rout = [torch.zeros(max(1, int(counts[r])), device="cuda") for r in range(p)]
    c.reduce_scatter_v(rin, rout, counts, displs, algo=L.ALGO_RING)
    ok(c)
    ref = ref_reduce(rin, L.SUM)
    for r in range(p):
        close(rout[r][:int(counts[r])], ref[int(displs[r]):int(displs[r] + counts[r])], torch.float32, p)
    c.barrier()
    ok(c)
    a = torch.randn(200_000, device="cuda")
    b = torch.zeros_like(a)
    c.local_send_recv(0, 2, a, b)
    ok(c)
    assert torch.equal(a, b)


def test_bounded_wait_reports_timeout_and_recovers():
    """A wait for a flag that nothing sets must end after its bound with HCCL_E_TIMEOUT in the host-visible status
    block, the CUDA context must stay usable, and the communicator must work again after resume."""
    import time
    cfg = L.CommConfig.default()
    cfg.hcclBufferSize = 1
    c = H.Communicator.init_local(2, device=True, device_id=0, config=cfg)
    x = [torch.ones(1024, device="cuda") for _ in range(2)]
    y = [torch.zeros(1024, device="cuda") for _ in range(2)]
    c.all_reduce(x, y)
    assert c.sync() == 0
    t0 = time.time()
    assert c.wait_probe(0, timeout_ms=300.0) == L.E_TIMEOUT
    assert 0.25 < time.time() - t0 < 5.0
    st = c.status(0)
    assert st.code == L.E_TIMEOUT and st.peer == 1 and st.seen < st.expected
    assert "waiting for rank 1" in c.describe_status(0)
    with pytest.raises(H.HcclError) as e:
        c.all_reduce(x, y)  # refused until resumed
    assert e.value.code == L.E_TIMEOUT
    c.resume()
    c.all_reduce(x, y)
    assert c.sync() == 0 and torch.all(y[0] == 2)
    # suspend: the abort word refuses new work; resume re-arms
    c.suspend()
    with pytest.raises(H.HcclError) as e:
        c.all_reduce(x, y)
    assert e.value.code == L.E_SUSPENDING
    c.resume()
    c.all_reduce(x, y)
    assert c.sync() == 0
    assert float(torch.ones(4, device="cuda").sum()) == 4.0  # context still healthy
    c.destroy()


def test_single_rank_c_api_and_stats():
    c = H.Communicator.init_root(1, H.Communicator.get_root_info(), 0, device=True)
    x = torch.randn(1 << 18, device="cuda")
    y = torch.zeros_like(x)
    c.all_reduce(x, y)
    ok(c)
    assert torch.equal(x, y)
    g = torch.zeros_like(x)
    c.all_gather(x, g)
    ok(c)
    assert torch.equal(x, g)
    st = c.stats()
    assert st["launches"] >= 2 and st["ops"]["AllReduce"]["calls"] == 1
    c.destroy()


def test_one_sided_topology_overflow_device(comms, monkeypatch):
    """Put / get through peer mappings (copy engine), topology description, and the Inf / NaN scan after a reduction."""
    p = 4
    c = comms(p)
    n = 1024
    handle, bufs = c.symmetric_empty(n * p, torch.float32)
    for b in bufs:
        b.fill_(-1)
    torch.cuda.synchronize()
    srcs = [torch.full((n,), float(r + 1), device="cuda") for r in range(p)]
    for r in range(p):          # virtual rank r writes its block into slot r of every rank's copy
        for q in range(p):
            c.put(handle, q, r * n * 4, srcs[r].data_ptr(), n * 4, local=r)
    torch.cuda.synchronize()
    want = torch.arange(1, p + 1, device="cuda", dtype=torch.float32).repeat_interleave(n)
    for b in bufs:
        assert torch.equal(b, want)
    got = torch.zeros(n, device="cuda")
    c.get(handle, 2, 2 * n * 4, got.data_ptr(), n * 4, local=1)
    torch.cuda.synchronize()
    assert torch.equal(got, torch.full((n,), 3.0, device="cuda"))
    with pytest.raises(H.HcclError):
        c.put(handle, 0, n * p * 4, srcs[0].data_ptr(), 16)
    del bufs, b
    c.mem_free(handle)
    topo = c.topology()
    assert topo["ranks"] == p and topo["transport"] == "device" and topo["all_local"] and topo["peer_access"] == [[1]]
    td = c.topo_desc()
    assert td[0][1] == p and td[0][0] & L.ALG_MESH and td[1] == (0, 0)
    monkeypatch.setenv("HCCL_OVERFLOW_CHECK", "1")
    L.lib().HcclB200ReloadEnv()
    try:
        xs = [torch.ones(5000, device="cuda", dtype=torch.bfloat16) for _ in range(p)]
        ys = [torch.empty_like(x) for x in xs]
        c.all_reduce(xs, ys)
        ok(c)
        assert c.overflow_count() == 0
        xs[1][17] = float("inf")
        xs[2][99] = float("nan")
        c.all_reduce(xs, ys)
        ok(c)
        assert c.overflow_count() == 2 * p      # two bad outputs on each of the p virtual ranks
    finally:
        monkeypatch.delenv("HCCL_OVERFLOW_CHECK")
        L.lib().HcclB200ReloadEnv()
