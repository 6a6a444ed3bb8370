"""MoE dispatch / combine on symmetric memory (virtual ranks of one GPU) against the plain PyTorch statement."""
import pytest

torch = pytest.importorskip("torch")
import cann_hccl_b200 as H  # noqa: E402
from cann_hccl_b200 import _lib as L  # noqa: E402
from cann_hccl_b200.parallel import moe  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("p", [1, 2, 4])
@pytest.mark.parametrize("variant", ["mesh", "pairwise"])
def test_dispatch_combine(p, variant):
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    cfg = L.CommConfig.default()
    cfg.hcclBufferSize = 2
    c = H.Communicator.init_local(p, device=True, device_id=0, config=cfg)
    T, Hd, E, k = 96, 256, 8 * p, 2
    ex = moe.MoEExchange(c, T, Hd, E, k, capacity_factor=float(p) * 1.0 + 0.5)
    xs = [torch.randn(T, Hd, device="cuda").to(torch.bfloat16) for _ in range(p)]
    routed = [moe.route(T, E, k, 7, r) for r in range(p)]
    idx, gates = [r[0] for r in routed], [r[1] for r in routed]
    one = p == 1
    for _ in range(2):
        recv, offs, rows = ex.dispatch(xs[0] if one else xs, idx[0] if one else idx, variant=variant)
        assert c.sync() == 0, c.describe_status()
        recv, offs, rows = ([recv], [offs], [rows]) if one else (recv, offs, rows)
        El = E // p
        # receive side: rows grouped by local expert; the multiset of rows per expert equals what was routed there
        for r in range(p):
            assert int(ex.overflow[r].item()) == 0
            o = offs[r].tolist()
            assert o[-1] == int(rows[r].item())
            for el in range(El):
                e = r * El + el
                want = torch.cat([xs[s][(idx[s] == e).any(dim=1)] for s in range(p)]) if True else None
                got = recv[r][o[el]:o[el + 1]]
                assert got.shape[0] == want.shape[0]
                assert torch.equal(got.float().sum(0), got.float().sum(0))
                # order inside (source, expert) groups is arrival order: compare as multisets via sorting by row sums
                ks = lambda t: t[torch.argsort(t.float().sum(1))]
                assert torch.allclose(ks(got).float(), ks(want).float())
            # "experts": scale rows by (1 + local expert id) so that combine has something to weight
            for el in range(El):
                ex.expert_out[r][o[el]:o[el + 1]] = (recv[r][o[el]:o[el + 1]].float() * (1 + r * El + el)).to(torch.bfloat16)
        outs = ex.combine(gates[0] if one else gates, variant=variant)
        assert c.sync() == 0, c.describe_status()
        outs = [outs] if one else outs
        for r in range(p):
            w = (gates[r] * (1 + idx[r].float())).sum(1, keepdim=True)          # sum_k gate * (1 + expert)
            want = xs[r].float() * w
            # expert outputs were rounded to bf16 once: tolerance of one bf16 ulp on the scaled rows
            assert torch.allclose(outs[r].float(), want, rtol=2e-2, atol=2e-2)
    ex.close()
    c.destroy()
