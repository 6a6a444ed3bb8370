"""Mapping between numpy / torch dtypes and HcclDataType."""
import numpy as np

from .. import _lib as L

_NP = {np.dtype("int8"): L.INT8, np.dtype("int16"): L.INT16, np.dtype("int32"): L.INT32, np.dtype("float16"): L.FP16,
       np.dtype("float32"): L.FP32, np.dtype("int64"): L.INT64, np.dtype("uint64"): L.UINT64, np.dtype("uint8"): L.UINT8,
       np.dtype("uint16"): L.UINT16, np.dtype("uint32"): L.UINT32, np.dtype("float64"): L.FP64}


def _torch_map():
    import torch
    m = {torch.int8: L.INT8, torch.int16: L.INT16, torch.int32: L.INT32, torch.float16: L.FP16, torch.float32: L.FP32,
         torch.int64: L.INT64, torch.uint8: L.UINT8, torch.float64: L.FP64, torch.bfloat16: L.BFP16}
    for name, code in (("uint16", L.UINT16), ("uint32", L.UINT32), ("uint64", L.UINT64), ("float8_e4m3fn", L.FP8E4M3),
                       ("float8_e5m2", L.FP8E5M2)):
        if hasattr(torch, name):
            m[getattr(torch, name)] = code
    return m


_TORCH = None


def hccl_dtype(x):
    """HcclDataType of a numpy array or torch tensor."""
    global _TORCH
    if isinstance(x, np.ndarray):
        return _NP[x.dtype]
    if _TORCH is None:
        _TORCH = _torch_map()
    return _TORCH[x.dtype]


def data_ptr(x):
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    return x.data_ptr()


def numel(x):
    return int(x.size) if isinstance(x, np.ndarray) else int(x.numel())


def is_device(x):
    return (not isinstance(x, np.ndarray)) and x.is_cuda
