"""tcgen05 GEMM and the fused GEMM + collective kernels against a plain PyTorch fp32 reference.
Multi-rank cases run as virtual ranks of one GPU (one cooperative launch, peers = other buffers of the same device)."""
import pytest

torch = pytest.importorskip("torch")
import cann_hccl_b200 as H  # noqa: E402
from cann_hccl_b200 import _lib as L  # noqa: E402
from cann_hccl_b200.parallel import fused_tp  # noqa: E402

pytestmark = pytest.mark.gpu


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")


def rel_err(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 128), (512, 1024, 4096), (2048, 768, 320)])
def test_gemm_bf16(M, N, K):
    _need_gpu()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    c = fused_tp.gemm(a, b)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    assert rel_err(c, ref) < 1e-2
    # a second shape-identical call reuses the pipeline state machine from scratch
    c2 = fused_tp.gemm(a, b)
    torch.cuda.synchronize()
    assert torch.equal(c, c2)


def test_gemm_bf16_every_tile_multi_wave():
    """2048 x 3584 x 8192: 224 output tiles of 128 x 256 on 148 SMs (more than one wave).  A global norm would hide one wrong
    tile, so every tile is held to a max-abs bound of its own against the fp32 product of the same bf16 operands."""
    _need_gpu()
    M, N, K = 2048, 3584, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    c = fused_tp.gemm(a, b)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().view(M // 128, 128, N // 256, 256).amax(dim=(1, 3))      # [m tiles, n tiles]
    scale = ref.abs().view(M // 128, 128, N // 256, 256).amax(dim=(1, 3))
    # bf16 output rounding is 2^-8 relative; fp32 accumulation over K = 8192 adds far less
    bad = (err > scale * 2 ** -7).nonzero()
    assert bad.numel() == 0, "tiles off: %s (err %s)" % (bad[:8].tolist(), err[err > scale * 2 ** -7][:8].tolist())


def test_gemm_rejects_bad_shapes():
    _need_gpu()
    a = torch.zeros(100, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(H.HcclError):
        fused_tp.gemm(a, b)


@pytest.fixture(scope="module")
def comms():
    _need_gpu()
    cache = {}

    def get(p):
        if p not in cache:
            cfg = L.CommConfig.default()
            cfg.hcclBufferSize = 2
            cache[p] = H.Communicator.init_local(p, device=True, device_id=0, config=cfg)
        return cache[p]

    yield get
    for c in cache.values():
        assert c.destroy() == L.SUCCESS


@pytest.mark.parametrize("p", [1, 2, 4])
def test_all_gather_matmul(comms, p):
    c = comms(p)
    Ms, K, N = 256, 512, 512
    g = torch.Generator(device="cuda").manual_seed(p)
    xs = [torch.randn(Ms, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(p)]
    ws = [(torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16) for _ in range(p)]
    for _ in range(3):  # epochs of the workspace flags advance call by call
        ys = fused_tp.all_gather_matmul(c, xs if p > 1 else xs[0], ws if p > 1 else ws[0])
        assert c.sync() == 0, c.describe_status()
    ys = ys if p > 1 else [ys]
    xfull = torch.cat([x.float() for x in xs])
    for r in range(p):
        assert rel_err(ys[r], xfull @ ws[r].float().t()) < 1e-2


@pytest.mark.parametrize("p", [2, 4])
def test_all_gather_matmul_registered_source(comms, p):
    """Shards in registered symmetric memory are pulled by the peers where they lie (no staging copy); the caller may
    rewrite its shard right after the call, and an unregistered call on the same workspace may follow."""
    c = comms(p)
    Ms, K, N = 256, 512, 512
    g = torch.Generator(device="cuda").manual_seed(40 + p)
    handle, bufs = c.symmetric_empty(Ms * K, torch.bfloat16)
    xs = [b.view(Ms, K) for b in bufs]
    ws = [(torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16) for _ in range(p)]
    for it in range(3):
        vals = [torch.randn(Ms, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(p)]
        for x, v in zip(xs, vals):
            x.copy_(v)
        ys = fused_tp.all_gather_matmul(c, xs, ws)
        for x in xs:
            x.zero_()  # stream order: the kernel has let go of the shards by the time it ends
        assert c.sync() == 0, c.describe_status()
        xfull = torch.cat([v.float() for v in vals])
        for r in range(p):
            assert rel_err(ys[r], xfull @ ws[r].float().t()) < 1e-2
    plain = [v.clone() for v in vals]
    ys = fused_tp.all_gather_matmul(c, plain, ws)
    assert c.sync() == 0, c.describe_status()
    for r in range(p):
        assert rel_err(ys[r], xfull @ ws[r].float().t()) < 1e-2
    del xs, bufs
    c.mem_free(handle)


def test_all_gather_matmul_adopted_source(comms):
    """Ordinary tensors registered with mem_adopt are pulled in place like library-allocated symmetric memory."""
    p = 2
    c = comms(p)
    Ms, K, N = 256, 512, 512
    g = torch.Generator(device="cuda").manual_seed(77)
    xs = [torch.randn(Ms, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(p)]
    ws = [(torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16) for _ in range(p)]
    handle = c.mem_adopt(xs)
    table, _, nbytes = c.mem_query(handle)
    assert nbytes == Ms * K * 2 and table[0][1] == xs[1].data_ptr() and table[1][0] == xs[0].data_ptr()
    for _ in range(2):
        ys = fused_tp.all_gather_matmul(c, xs, ws)
        assert c.sync() == 0, c.describe_status()
    xfull = torch.cat([x.float() for x in xs])
    for r in range(p):
        assert rel_err(ys[r], xfull @ ws[r].float().t()) < 1e-2
    c.mem_free(handle)
    ys = fused_tp.all_gather_matmul(c, xs, ws)  # staged again
    assert c.sync() == 0, c.describe_status()
    for r in range(p):
        assert rel_err(ys[r], xfull @ ws[r].float().t()) < 1e-2


@pytest.mark.parametrize("p", [1, 2, 4])
def test_matmul_reduce_scatter(comms, p):
    c = comms(p)
    M, K, N = 256 * p, 256, 512
    g = torch.Generator(device="cuda").manual_seed(10 + p)
    hs = [torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(p)]
    ws = [(torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16) for _ in range(p)]
    for _ in range(3):
        outs = fused_tp.matmul_reduce_scatter(c, hs if p > 1 else hs[0], ws if p > 1 else ws[0])
        assert c.sync() == 0, c.describe_status()
    outs = outs if p > 1 else [outs]
    full = sum(h.float() @ w.float().t() for h, w in zip(hs, ws))
    rows = M // p
    for r in range(p):
        assert rel_err(outs[r], full[r * rows:(r + 1) * rows]) < 2e-2


def test_matmul_reduce_scatter_same_shape_other_depth_and_after_rejected_call(comms):
    """The completion-counter layout depends on K (wide K makes the panels narrower), so calls that share M and N but not K
    must not share counters; and a call rejected for its arguments must leave the workspace's call count alone."""
    p = 2
    c = comms(p)
    M, N = 512, 512
    g = torch.Generator(device="cuda").manual_seed(90)
    ws_small = None
    for K in (256, 20480, 256):
        hs = [torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16) for _ in range(p)]
        ws = [(torch.randn(N, K, device="cuda", generator=g) * 0.02).to(torch.bfloat16) for _ in range(p)]
        outs = fused_tp.matmul_reduce_scatter(c, hs, ws)
        assert c.sync() == 0, c.describe_status()
        full = sum(h.float() @ w.float().t() for h, w in zip(hs, ws))
        for r in range(p):
            assert rel_err(outs[r], full[r * (M // p):(r + 1) * (M // p)]) < 2e-2
        if K == 256:
            ws_small = (hs, ws, full)
    hs, ws, full = ws_small
    bad = [h[:, :200].contiguous() for h in hs]          # K = 200 is not a multiple of 64: refused before any launch
    with pytest.raises(H.HcclError):
        fused_tp.matmul_reduce_scatter(c, bad, [w[:, :200].contiguous() for w in ws])
    outs = fused_tp.matmul_reduce_scatter(c, hs, ws)     # the same workspace right after the refused call
    assert c.sync() == 0, c.describe_status()
    for r in range(p):
        assert rel_err(outs[r], full[r * (M // p):(r + 1) * (M // p)]) < 2e-2


def test_tensor_parallel_mlp_forward(comms):
    from cann_hccl_b200.models.tp_mlp import TensorParallelMLP
    p = 2
    c = comms(p)
    mlp = TensorParallelMLP(c, hidden=512, ffn=1024, seed=3)
    xs = [torch.randn(128, 512, device="cuda").to(torch.bfloat16) for _ in range(p)]
    ys = mlp.forward(xs)
    assert c.sync() == 0, c.describe_status()
    ref = mlp.reference_forward(xs)
    for got, want in zip(ys, ref):
        assert rel_err(got, want) < 3e-2


def test_zz_pair_variant_was_used_unless_switched_off():
    """Shapes whose rows per rank come in multiples of 256 run on clusters of two CTAs; HCCL_TP_GEMM_PAIR=0 keeps every
    launch on single CTAs."""
    import ctypes as C
    import os
    _need_gpu()
    single, pair = C.c_uint64(0), C.c_uint64(0)
    L.check(L.lib().HcclB200GemmLaunchCounts(C.byref(single), C.byref(pair)), "HcclB200GemmLaunchCounts")
    if os.environ.get("HCCL_TP_GEMM_PAIR") == "0":
        assert pair.value == 0 and single.value > 0, (single.value, pair.value)
    else:
        assert pair.value > 0 and single.value > 0, (single.value, pair.value)


def test_zzz_whole_file_again_on_single_ctas():
    """Runs this file once more in a child process with the pair variant switched off (one CTA per 128 x 256 tile, tcgen05
    cta_group::1): same shapes, same references."""
    import os
    import subprocess
    import sys
    _need_gpu()
    if os.environ.get("HCCL_TP_GEMM_PAIR") == "0":
        pytest.skip("already the single-CTA run")
    env = dict(os.environ, HCCL_TP_GEMM_PAIR="0")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-x", "-q", "-m", "gpu"], env=env, capture_output=True, text=True,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))), timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-1500:]
