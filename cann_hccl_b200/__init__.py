"""cann_hccl_b200: a Blackwell-native collective communication library with the HCCL C API.

Native code lives in csrc/ (built by `python -m cann_hccl_b200.build` into lib/libhccl_b200.so); this package is the
thin Python face: `Communicator` (ops/), fused tensor-parallel and MoE layers (parallel/), reference model blocks
that use them (models/) and helpers (utils/).
"""
from . import _lib  # noqa: F401
from ._lib import (ALGO_AUTO, ALGO_MESH, ALGO_MESH_ONESHOT, ALGO_NVLS, ALGO_NVLS_ONESHOT, ALGO_PAIRWISE, ALGO_RHD,  # noqa: F401
                   ALGO_RING, ALGO_STAR, ALGO_TREE, MAX, MIN, PROD, SUM, HcclError)
from .ops.comm import Communicator  # noqa: F401

__version__ = "0.1.0"
