"""ctypes binding of `libfluxb.so` (the C ABI declared in `include/fluxb.h`).

The library is the product: there is no Python or CPU fallback. If it is
missing it is built with nvcc; if that is impossible, importing fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

FLUXB_OK = 0
FLUXB_ERR_INVALID = -1
FLUXB_ERR_CUDA = -2
FLUXB_ERR_TIMEOUT = -3
FLUXB_ERR_UNSUPPORTED = -4
MAX_WORLD = 8
STATIC_MAX_ROWS = 65536
STATIC_MAX_EXPERTS = 256
IPC_HANDLE_BYTES = 64

BF16, F16, F32, E4M3, E5M2, S8 = 0, 1, 2, 3, 4, 5
BIAS_NONE, BIAS_MN, BIAS_1N = 0, 1, 2
WEIGHT_KN = 1
RS_FP32_WIRE = 2
RS_RING_ORDER = 4

STATUS_NAMES = {
    0: "ok",
    1: "timeout: operand stage never filled (TMA)",
    2: "timeout: operand stage never drained (MMA)",
    3: "timeout: accumulator never completed",
    4: "timeout: accumulator never drained",
    5: "timeout: a peer's arrival flag never reached its value",
    6: "timeout: all-rank barrier",
    7: "timeout: reduce-scatter partial tiles missing",
    8: "grouped GEMM: inconsistent tile table",
}


class Tuning(C.Structure):
    _fields_ = [("block_n", C.c_int), ("group_m", C.c_int), ("num_ctas", C.c_int), ("cta_group", C.c_int),
                ("ag_mode", C.c_int)]


TUNING_FIELDS = ("block_n", "group_m", "num_ctas", "cta_group", "ag_mode")
AG_MODE_KERNEL_PUSH, AG_MODE_COPY_ENGINE = 1, 2


def make_tuning(t) -> "Tuning":
    """A `Tuning` from a dict of its fields (missing fields = 0 = the library's choice)."""
    return Tuning(*[int(t.get(f, 0)) for f in TUNING_FIELDS])


class FluxbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"fluxb error {code}: {msg}")
        self.code = code


_vp = C.c_void_p
_i = C.c_int
_f = C.c_float
_sz = C.c_size_t
_pp = C.POINTER(C.c_void_p)
_tun = C.POINTER(Tuning)

# name -> (restype, argtypes); every symbol include/fluxb.h declares
SIGNATURES = {
    "fluxb_last_error": (C.c_char_p, []),
    "fluxb_version": (_i, []),
    "fluxb_device_supported": (_i, []),
    "fluxb_comm_create": (_i, [_i, _i, _pp]),
    "fluxb_comm_destroy": (_i, [_vp]),
    "fluxb_comm_set_timeout_ms": (_i, [_vp, _i]),
    "fluxb_comm_set_trace": (_i, [_vp, _vp]),
    "fluxb_status_peek": (_i, [_vp, C.POINTER(_i)]),
    "fluxb_status_clear": (_i, [_vp]),
    "fluxb_symm_alloc": (_i, [_sz, _pp, _vp]),
    "fluxb_symm_free": (_i, [_vp]),
    "fluxb_symm_open": (_i, [_vp, _pp]),
    "fluxb_symm_close": (_i, [_vp]),
    "fluxb_enable_peer_access": (_i, [_i, _i]),
    "fluxb_barrier_all": (_i, [_vp, _pp, _vp]),
    "fluxb_comm_set_ranks_on_gpu": (_i, [_vp, _i]),
    "fluxb_run_ranks": (_i, [_pp, _i, _vp]),
    "fluxb_gemm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp, _vp, _f, _i, _tun, _vp]),
    "fluxb_ag_gemm_gather_bytes": (_sz, [_i, _i, _i]),
    "fluxb_ag_gemm_flag_bytes": (_sz, [_i, _i]),
    "fluxb_ag_gemm_scale_bytes": (_sz, [_i]),
    "fluxb_ag_gemm_create": (_i, [_vp, _i, _i, _i, _i, _i, _pp, _pp, _pp, _pp]),
    "fluxb_ag_gemm_destroy": (_i, [_vp]),
    "fluxb_ag_gemm_reset": (_i, [_vp, _vp]),
    "fluxb_ag_gemm_forward": (_i, [_vp, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _vp, _vp, _f, _i, _vp, _tun, _vp]),
    "fluxb_gemm_rs_stage_bytes": (_sz, [_i, _i, _i]),
    "fluxb_gemm_rs_cnt_bytes": (_sz, [_i, _i, _i]),
    "fluxb_gemm_rs_create": (_i, [_vp, _i, _i, _i, _i, _pp, _pp, _pp]),
    "fluxb_gemm_rs_destroy": (_i, [_vp]),
    "fluxb_gemm_rs_reset": (_i, [_vp, _vp]),
    "fluxb_gemm_rs_forward": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _f, _i, _tun, _vp]),
    "fluxb_moe_scatter_index": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "fluxb_moe_gather_index": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "fluxb_moe_ag_scatter_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "fluxb_moe_ag_scatter_create": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _pp, _pp, _vp, _pp]),
    "fluxb_moe_ag_scatter_destroy": (_i, [_vp]),
    "fluxb_moe_ag_scatter_reset": (_i, [_vp, _vp]),
    "fluxb_moe_ag_scatter_set_ep": (_i, [_vp, _i, _i]),
    "fluxb_moe_ag_scatter_forward": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _tun, _vp]),
    "fluxb_moe_scatter_gemm_static": (_i, [_vp, _vp, _i, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _tun, _vp]),
    "fluxb_moe_gather_rs_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "fluxb_moe_gather_rs_stage_bytes": (_sz, [_i, _i, _i, _i]),
    "fluxb_moe_gather_rs_cnt_bytes": (_sz, [_i, _i, _i, _i]),
    "fluxb_moe_gather_rs_create": (_i, [_vp, _i, _i, _i, _i, _i, _i, _pp, _pp, _vp, _pp]),
    "fluxb_moe_gather_rs_destroy": (_i, [_vp]),
    "fluxb_moe_gather_rs_reset": (_i, [_vp, _vp]),
    "fluxb_moe_gather_rs_forward": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _tun, _vp]),
    "fluxb_moe_gather_rs_set_ep": (_i, [_vp, _i, _i]),
    "fluxb_moe_gather_rs_forward_ep": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _tun, _vp]),
}

_LIB = None


def lib_path() -> Path:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Load (building first if needed) the native library and type its entry points."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists() or os.environ.get("FLUXB_REBUILD") == "1":
        _build.build_library(force=True)
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def last_error() -> str:
    return load().fluxb_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != FLUXB_OK:
        raise FluxbError(rc, last_error())


def ptr_table(ptrs) -> C.Array:
    arr = (C.c_void_p * MAX_WORLD)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr
