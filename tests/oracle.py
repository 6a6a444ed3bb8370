"""Single-process numpy reference of every collective (hccl_test `check_result` semantics)."""
import numpy as np

from cann_hccl_b200 import _lib as L


def np_reduce(arrs, op):
    acc_dtype = np.float32 if arrs[0].dtype == np.float16 else arrs[0].dtype
    acc = arrs[0].astype(acc_dtype)
    for a in arrs[1:]:
        b = a.astype(acc_dtype)
        if op == L.SUM:
            acc = acc + b
        elif op == L.PROD:
            acc = acc * b
        elif op == L.MAX:
            acc = np.maximum(acc, b)
        else:
            acc = np.minimum(acc, b)
    return acc.astype(arrs[0].dtype)


def tol(dtype, p):
    if dtype == np.float32:
        return dict(rtol=1e-6 * p, atol=1e-6 * p)
    if dtype == np.float16:
        return dict(rtol=4e-3, atol=4e-3 * p)
    if dtype == np.float64:
        return dict(rtol=1e-12 * p, atol=1e-12 * p)
    return dict(rtol=0, atol=0)


def make_inputs(p, n, dtype, seed=1234):
    out = []
    for r in range(p):
        rng = np.random.default_rng(seed + r)
        if np.issubdtype(dtype, np.floating):
            out.append(rng.uniform(-1, 1, n).astype(dtype))
        elif np.issubdtype(dtype, np.unsignedinteger):
            out.append(rng.integers(0, 5, n).astype(dtype))
        else:
            out.append(rng.integers(-3, 4, n).astype(dtype))
    return out
