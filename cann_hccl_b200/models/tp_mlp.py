"""Tensor-parallel MLP block (Llama-style shapes) built on the fused kernels.

The activations enter and leave sharded by rows (sequence-parallel layout): each rank holds [tokens/p, hidden].
    h = act( all_gather(x) @ W_up[ffn/p, hidden].T )      one fused all-gather + GEMM kernel
    y = reduce_scatter( h @ W_down[hidden, ffn/p].T )     one fused GEMM + reduce-scatter kernel
Weights are random (N(0, 0.02)); `reference_forward` is the plain PyTorch fp32 statement of the same math.
"""
import torch

from ..parallel import fused_tp


class TensorParallelMLP:
    def __init__(self, comm, hidden, ffn, seed=0, activation="silu", device="cuda"):
        self.comm, self.hidden, self.ffn = comm, hidden, ffn
        p = comm.nranks
        assert ffn % p == 0
        self.act = {"silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu, "none": lambda t: t}[activation]
        g = torch.Generator(device=device).manual_seed(seed)
        # full weights are generated identically on every rank, then sliced: rank r owns rows / columns [r*ffn/p, (r+1)*ffn/p)
        w_up = (torch.randn(ffn, hidden, device=device, generator=g) * 0.02).to(torch.bfloat16)
        w_down = (torch.randn(hidden, ffn, device=device, generator=g) * 0.02).to(torch.bfloat16)
        self.w_up_full, self.w_down_full = w_up, w_down
        fs = ffn // p
        ranks = range(p) if comm.nlocal > 1 else [comm.rank]
        self.w_up = [w_up[r * fs:(r + 1) * fs].contiguous() for r in ranks]
        self.w_down = [w_down[:, r * fs:(r + 1) * fs].contiguous() for r in ranks]

    def forward(self, x_shards):
        """x_shards: this rank's [tokens/p, hidden] tensor (or a list, one per virtual rank)."""
        single = not isinstance(x_shards, (list, tuple))
        xs = [x_shards] if single else list(x_shards)
        h = fused_tp.all_gather_matmul(self.comm, xs if not single else xs[0], self.w_up if not single else self.w_up[0])
        hs = [h] if single else h
        hs = [self.act(t.float()).to(torch.bfloat16) for t in hs]
        y = fused_tp.matmul_reduce_scatter(self.comm, hs if not single else hs[0], self.w_down if not single else self.w_down[0])
        return y

    def reference_forward(self, all_x_shards):
        """fp32 PyTorch reference given every rank's shard (list of p tensors); returns the p output shards."""
        x = torch.cat([t.float() for t in all_x_shards], dim=0)
        h = self.act(x @ self.w_up_full.float().t()).to(torch.bfloat16).float()
        y = h @ self.w_down_full.float().t()
        p = len(all_x_shards)
        rows = y.shape[0] // p
        return [y[r * rows:(r + 1) * rows].to(torch.bfloat16) for r in range(p)]
