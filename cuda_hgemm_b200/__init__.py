"""B200-native half-precision GEMM: hand-written sm_100a kernels behind a C ABI.

The package holds the native sources (``csrc/``), their build recipe (``build.py``), the
ctypes binding of the C ABI (``_native.py``), thin torch-tensor wrappers with the reference's
entry-point convention (``api.py``) and the row-slab partitioner used when a GEMM is spread
over several GPUs (``partition.py``).
"""
from .api import *  # noqa: F401,F403
from .api import __all__ as _api_all
from .partition import row_slabs  # noqa: F401

__all__ = list(_api_all) + ["row_slabs"]
