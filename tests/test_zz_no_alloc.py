"""The allocation-free entry point `hcclb200_matmul_reduce_noalloc`, called through its exported C symbol.

Some callers of the row-parallel GEMM cannot allocate device memory when they call it (they run inside another
allocator's callback, in a latency-critical loop, or after all free memory went to a pool), so that entry point keeps
its scratch (receive slot + completion counters) in a fixed device array inside the library.  Its result must equal
the result of the ordinary entry point (HcclB200MatmulReduceScatter on a one-rank communicator, whose scratch comes
from the communicator's symmetric heap) — on the first call, which sets the device up, and on a second call, which
finds the array as the first call left it.  This file is collected last on purpose.
"""
import ctypes as C

import pytest

torch = pytest.importorskip("torch")
import cann_hccl_b200 as H  # noqa: E402
from cann_hccl_b200 import _lib as L  # noqa: E402
from cann_hccl_b200.parallel import fused_tp  # noqa: E402

pytestmark = pytest.mark.gpu


def test_no_alloc_entry_matches_regular_entry_twice():
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    lib = L.lib()
    fn = lib.hcclb200_matmul_reduce_noalloc
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    status = lib.hcclb200_matmul_reduce_noalloc_status
    status.argtypes = [C.c_void_p]
    status.restype = C.c_int
    comm = H.Communicator.init_root(1, H.Communicator.get_root_info(), 0, device=True)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (M, N, K) in enumerate([(512, 1024, 256), (1024, 2048, 512)]):
        g = torch.Generator(device="cuda").manual_seed(call)
        h = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
        want = fused_tp.matmul_reduce_scatter(comm, h, w)             # existing entry point
        assert comm.sync() == 0, comm.describe_status()
        got = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(h.data_ptr(), w.data_ptr(), got.data_ptr(), M, N, K, stream)
        assert rc == 0, rc
        assert status(stream) == 0                                     # no bounded wait of the kernel ran out (also waits for the stream)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before            # nothing was allocated on the device
        # same kernel, same arithmetic: the tolerance of the fused-kernel tests (relative Frobenius error)
        err = float((got.float() - want.float()).norm() / want.float().norm())
        assert err < 1e-2, err
        ref = h.float() @ w.float().t()
        assert float((got.float() - ref).norm() / ref.norm()) < 1e-2
    # sizes beyond the built-in scratch are refused before anything is launched
    big = torch.empty(8, device="cuda", dtype=torch.bfloat16)
    assert fn(big.data_ptr(), big.data_ptr(), big.data_ptr(), 2048, 2048, 64, stream) == L.E_MEMORY
    assert fn(big.data_ptr(), big.data_ptr(), big.data_ptr(), 100, 256, 64, stream) == L.E_PARA
    assert fn(None, big.data_ptr(), big.data_ptr(), 128, 256, 64, stream) == L.E_PTR
    comm.destroy()
