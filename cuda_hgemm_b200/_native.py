"""ctypes binding of the C ABI declared in ``include/b200_hgemm.h``.

The shared library is built in-tree (``cuda_hgemm_b200/lib/libb200_hgemm.so``). There is no
fallback of any kind: if the library is missing, loading raises, and every compute call on a
device that is not sm_100 returns an error code that ``check()`` turns into an exception.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libb200_hgemm.so"

# every symbol include/b200_hgemm.h declares
EXPORTED_SYMBOLS = (
    "b200_hgemm", "b200_hgemm_cta1", "b200_hgemm_cta2", "b200_hgemm_splitk", "b200_hgemm_streamk",
    "b200_hgemm_simt", "b200_hgemm_streamk_static", "b200_hgemm_ex", "b200_hgemm_host", "b200_hgemm_select", "b200_hgemm_workspace_bytes",
    "b200_hgemm_set_workspace", "b200_hgemm_last_device_error", "b200_hgemm_status_string",
    "b200_hgemm_version", "b200_hgemm_launch_count", "b200_sched_tile_coord", "b200_sched_segments",
    "b200_sched_contributors", "b200_sched_partial_slot", "b200_debug_idesc", "b200_debug_smem_desc",
    "b200_debug_wait_expiry", "b200_hgemm_fused", "b200_hgemm_host_a", "b200_hgemm_load_plan_table", "b200_hgemm_select_untuned", "b200_partition_slab", "b200_mg_create", "b200_mg_destroy", "b200_mg_device_count",
    "b200_mg_slab", "b200_mg_hgemm", "b200_mg_gather_c", "b200_mg_synchronize", "b200_mg_elapsed_ms_max",
    "b200_hgemm_enable_multicast", "b200_hgemm_multicast_state", "b200_hgemm_plan_supported",
    "b200_hgemm_release_workspaces", "b200_hgemm_synchronize", "b200_hgemm_streamk_static_last_error",
    "b200_debug_wait_expiry_static", "b200_hgemm_fused_ex", "b200_hgemm_batched", "b200_hgemm_bkn", "b200_hgemm_host_a_after", "b200_sched_tile_coord_fast", "b200_debug_fast_div", "b200_debug_cluster_capacity",
)

OK = 0
ERR_INVALID_ARG = -1
ERR_UNSUPPORTED = -2
ERR_MISALIGNED = -3
ERR_NO_SM100 = -4
ERR_CUDA = -5
ERR_WORKSPACE = -6
ERR_DEVICE_WAIT = -7
ERR_TOO_LARGE = -8

VARIANT_CTA1 = 0
VARIANT_CTA2 = 1
VARIANT_STREAMK = 2
VARIANT_SIMT = 3
VARIANT_CTA2_MCAST = 4
VARIANT_SKINNY = 5
VARIANT_HYBRID = 6
VARIANT_SKINNY_PAIR = 7
VARIANT_HYBRID_PAIR = 8

C_F16, C_BF16, C_F32 = 0, 1, 2

MULTICAST_OFF, MULTICAST_ON, MULTICAST_LOCKED_OFF = 0, 1, 2


class Plan(Structure):
    """Mirror of ``b200_hgemm_plan``."""
    _fields_ = [("variant", c_int32), ("bn", c_int32), ("parts", c_int32), ("group_m", c_int32),
                ("tma_store", c_int32), ("grid", c_int32), ("stages", c_int32)]

    def as_dict(self):
        return {name: int(getattr(self, name)) for name, _ in self._fields_}


class Epilogue(Structure):
    """``b200_hgemm_epilogue``: C = alpha * A*B^T + beta * c_in + bias."""
    _fields_ = [("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("bias", c_void_p), ("c_in", c_void_p),
                ("c_type", c_int32)]


class HgemmError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200_hgemm status {status}: {message}")
        self.status = status


_lib = None


def load() -> ctypes.CDLL:
    """Load the native library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m cuda_hgemm_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(str(LIB_PATH))
    gemm_args = [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p]
    for name in ("b200_hgemm", "b200_hgemm_cta1", "b200_hgemm_cta2", "b200_hgemm_splitk", "b200_hgemm_streamk",
                 "b200_hgemm_simt", "b200_hgemm_streamk_static", "b200_hgemm_bkn"):
        fn = getattr(lib, name)
        fn.argtypes = gemm_args
        fn.restype = c_int
    lib.b200_hgemm_ex.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, POINTER(Plan), c_void_p]
    lib.b200_hgemm_ex.restype = c_int
    lib.b200_hgemm_fused.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, POINTER(Epilogue), c_void_p]
    lib.b200_hgemm_fused.restype = c_int
    lib.b200_hgemm_fused_ex.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, POINTER(Epilogue),
                                        POINTER(Plan), c_void_p]
    lib.b200_hgemm_fused_ex.restype = c_int
    lib.b200_hgemm_batched.argtypes = [c_void_p, c_void_p, c_void_p] + [c_size_t] * 7 + [c_void_p]
    lib.b200_hgemm_batched.restype = c_int
    lib.b200_hgemm_host.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t]
    lib.b200_hgemm_host.restype = c_int
    lib.b200_hgemm_host_a.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t]
    lib.b200_hgemm_host_a.restype = c_int
    lib.b200_hgemm_host_a_after.argtypes = [c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p]
    lib.b200_hgemm_host_a_after.restype = c_int
    lib.b200_hgemm_select.argtypes = [c_size_t, c_size_t, c_size_t, POINTER(Plan)]
    lib.b200_hgemm_select.restype = c_int
    lib.b200_hgemm_select_untuned.argtypes = [c_size_t, c_size_t, c_size_t, POINTER(Plan)]
    lib.b200_hgemm_select_untuned.restype = c_int
    lib.b200_hgemm_load_plan_table.argtypes = [c_char_p]
    lib.b200_hgemm_load_plan_table.restype = c_int
    lib.b200_hgemm_workspace_bytes.argtypes = [c_size_t, c_size_t, c_size_t, POINTER(Plan)]
    lib.b200_hgemm_workspace_bytes.restype = c_size_t
    lib.b200_hgemm_set_workspace.argtypes = [c_void_p, c_size_t]
    lib.b200_hgemm_set_workspace.restype = c_int
    lib.b200_hgemm_last_device_error.argtypes = []
    lib.b200_hgemm_last_device_error.restype = c_int
    lib.b200_hgemm_streamk_static_last_error.argtypes = []
    lib.b200_hgemm_streamk_static_last_error.restype = c_int
    lib.b200_hgemm_synchronize.argtypes = [c_void_p]
    lib.b200_hgemm_synchronize.restype = c_int
    lib.b200_hgemm_release_workspaces.argtypes = []
    lib.b200_hgemm_release_workspaces.restype = c_int
    lib.b200_hgemm_enable_multicast.argtypes = [c_int]
    lib.b200_hgemm_enable_multicast.restype = c_int
    lib.b200_hgemm_multicast_state.argtypes = []
    lib.b200_hgemm_multicast_state.restype = c_int
    lib.b200_hgemm_plan_supported.argtypes = [c_size_t, c_size_t, c_size_t, POINTER(Plan)]
    lib.b200_hgemm_plan_supported.restype = c_int
    lib.b200_hgemm_status_string.argtypes = [c_int]
    lib.b200_hgemm_status_string.restype = c_char_p
    lib.b200_hgemm_version.argtypes = []
    lib.b200_hgemm_version.restype = c_char_p
    lib.b200_hgemm_launch_count.argtypes = []
    lib.b200_hgemm_launch_count.restype = c_uint64
    lib.b200_sched_tile_coord.argtypes = [c_uint32, c_uint32, c_uint32, c_uint32, POINTER(c_uint32), POINTER(c_uint32)]
    lib.b200_sched_tile_coord.restype = None
    lib.b200_sched_tile_coord_fast.argtypes = [c_uint32, c_uint32, c_uint32, c_uint32, POINTER(c_uint32), POINTER(c_uint32)]
    lib.b200_sched_tile_coord_fast.restype = None
    lib.b200_debug_cluster_capacity.argtypes = [c_int]
    lib.b200_debug_cluster_capacity.restype = None
    lib.b200_debug_fast_div.argtypes = [c_uint32, c_uint32]
    lib.b200_debug_fast_div.restype = c_uint32
    lib.b200_sched_segments.argtypes = [c_uint32, c_uint32, c_uint32, c_uint32, POINTER(c_uint32), c_uint32]
    lib.b200_sched_segments.restype = c_uint32
    lib.b200_sched_contributors.argtypes = [c_uint32, c_uint32, c_uint32, c_uint32, POINTER(c_uint32), POINTER(c_uint32)]
    lib.b200_sched_contributors.restype = None
    lib.b200_sched_partial_slot.argtypes = [c_uint32, c_uint32, c_uint32, c_uint32, c_uint32]
    lib.b200_sched_partial_slot.restype = c_uint32
    lib.b200_debug_wait_expiry.argtypes = [c_uint32, c_void_p]
    lib.b200_debug_wait_expiry.restype = c_int
    lib.b200_debug_wait_expiry_static.argtypes = [c_uint32, c_void_p]
    lib.b200_debug_wait_expiry_static.restype = c_int
    lib.b200_partition_slab.argtypes = [c_size_t, c_int, c_int, POINTER(c_size_t), POINTER(c_size_t)]
    lib.b200_partition_slab.restype = c_int
    lib.b200_mg_create.argtypes = [POINTER(c_int), c_int, POINTER(c_void_p)]
    lib.b200_mg_create.restype = c_int
    lib.b200_mg_destroy.argtypes = [c_void_p]
    lib.b200_mg_destroy.restype = c_int
    lib.b200_mg_device_count.argtypes = [c_void_p]
    lib.b200_mg_device_count.restype = c_int
    lib.b200_mg_slab.argtypes = [c_void_p, c_size_t, c_int, POINTER(c_size_t), POINTER(c_size_t)]
    lib.b200_mg_slab.restype = c_int
    lib.b200_mg_hgemm.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), c_size_t, c_size_t, c_size_t]
    lib.b200_mg_hgemm.restype = c_int
    lib.b200_mg_gather_c.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_void_p), c_size_t, c_size_t]
    lib.b200_mg_gather_c.restype = c_int
    lib.b200_mg_synchronize.argtypes = [c_void_p]
    lib.b200_mg_synchronize.restype = c_int
    lib.b200_mg_elapsed_ms_max.argtypes = [c_void_p, POINTER(ctypes.c_float)]
    lib.b200_mg_elapsed_ms_max.restype = c_int
    lib.b200_debug_idesc.argtypes = [c_uint32, c_uint32]
    lib.b200_debug_idesc.restype = c_uint32
    lib.b200_debug_smem_desc.argtypes = [c_uint32]
    lib.b200_debug_smem_desc.restype = c_uint64
    _lib = lib
    return lib


def status_string(status: int) -> str:
    return load().b200_hgemm_status_string(status).decode()


def check(status: int) -> None:
    if status != OK:
        raise HgemmError(status, status_string(status))
