"""Fused tensor-parallel operators: tcgen05 GEMM and its NVLink collective in one sm_100a kernel.

    gemm(a, b)                               -> a @ b.T                       (bf16, no communication)
    all_gather_matmul(comm, x_shard, w)      -> all_gather_rows(x_shard) @ w.T   (column-parallel linear)
    matmul_reduce_scatter(comm, h, w)        -> reduce_scatter_rows(h @ w.T)     (row-parallel linear)

Weights use the nn.Linear layout [out_features, in_features].  On an all-local communicator every argument is a list
with one tensor per virtual rank.
"""
import ctypes as C

import torch

from .. import _lib as L
from ..ops.comm import _raw_stream


def _stream():
    return C.c_void_p(_raw_stream())


def _check(t, name):
    assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous(), "%s must be a contiguous CUDA bf16 tensor" % name


def gemm(a, b, out=None):
    """a [M, K] @ b[N, K].T -> [M, N] with the library's tcgen05 kernel (M % 128 == N % 256 == K % 64 == 0)."""
    _check(a, "a")
    _check(b, "b")
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=torch.bfloat16)
    L.check(L.lib().HcclB200GemmBf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, _stream()), "HcclB200GemmBf16")
    return out


def _lists(comm, *xs):
    out = []
    for x in xs:
        if comm.nlocal == 1 and not isinstance(x, (list, tuple)):
            x = [x]
        assert len(x) == comm.nlocal
        out.append(list(x))
    return out


def _ptrs(ts):
    return (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


def all_gather_matmul(comm, x_shard, w, out=None):
    xs, ws = _lists(comm, x_shard, w)
    for t in xs + ws:
        _check(t, "operand")
    Ms, K = xs[0].shape
    N = ws[0].shape[0]
    M = Ms * comm.nranks
    outs = _lists(comm, out)[0] if out is not None else [torch.empty((M, N), device=t.device, dtype=torch.bfloat16) for t in xs]
    L.check(L.lib().HcclB200AllGatherMatmul(comm.handle, _ptrs(xs), _ptrs(ws), _ptrs(outs), M, N, K, _stream()), "HcclB200AllGatherMatmul")
    return outs[0] if comm.nlocal == 1 else outs


def matmul_reduce_scatter(comm, h, w, out=None):
    hs, ws = _lists(comm, h, w)
    for t in hs + ws:
        _check(t, "operand")
    M, K = hs[0].shape
    N = ws[0].shape[0]
    outs = _lists(comm, out)[0] if out is not None else [torch.empty((M // comm.nranks, N), device=t.device, dtype=torch.bfloat16) for t in hs]
    L.check(L.lib().HcclB200MatmulReduceScatter(comm.handle, _ptrs(hs), _ptrs(ws), _ptrs(outs), M, N, K, _stream()), "HcclB200MatmulReduceScatter")
    return outs[0] if comm.nlocal == 1 else outs


def smoke():
    """Tiny forward of the tensor-parallel MLP on cuda:0: plain GEMM, then two virtual ranks through both fused kernels."""
    from ..models.tp_mlp import TensorParallelMLP
    from ..ops.comm import Communicator
    torch.manual_seed(0)
    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    c = gemm(a, b)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    assert torch.allclose(c.float(), ref, rtol=2e-2, atol=2e-1), "tcgen05 GEMM mismatch"
    cfg = L.CommConfig.default()
    cfg.hcclBufferSize = 4
    comm = Communicator.init_local(2, device=True, device_id=0, config=cfg)
    mlp = TensorParallelMLP(comm, hidden=256, ffn=512, seed=0)
    x = [torch.randn(128, 256, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    y = mlp.forward(x)
    assert comm.sync() == 0, comm.describe_status()
    ref = mlp.reference_forward(x)
    for got, want in zip(y, ref):
        assert torch.allclose(got.float(), want.float(), rtol=5e-2, atol=5e-1), "fused MLP mismatch"
    comm.destroy()
