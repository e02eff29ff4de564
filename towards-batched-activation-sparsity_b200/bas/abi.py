"""Loads ``libbas.so`` and declares the C ABI of ``include/bas.h`` for ctypes."""

from __future__ import annotations

import ctypes as C
from pathlib import Path

BLOCK_K = 64
TILE_N = 128
MAX_BATCH = 64
SCORE_NORM = 0
SCORE_ENERGY = 1
IDS_STABLE = 16          # BAS_GEMM_IDS_STABLE
X_STABLE = 64            # BAS_GEMM_X_STABLE
NEXT_INDEPENDENT = 128   # BAS_GEMM_NEXT_INDEPENDENT
GEMM_BF16 = 32           # BAS_GEMM_BF16
SCORE_BF16 = 256         # BAS_SCORE_BF16
SCORE_INPUTS_STABLE = 512   # BAS_SCORE_INPUTS_STABLE
TP_HANDLE_BYTES = 64     # BAS_TP_HANDLE_BYTES

LIST_MAX_BLOCKS = 1024  # BAS_LIST_MAX_BLOCKS
LIST_MAX_CALLS = 4096   # BAS_LIST_MAX_CALLS
DEV_BAD_BLOCK_ID = 1     # BAS_DEV_BAD_BLOCK_ID
DEV_WAIT_EXPIRED = 2     # BAS_DEV_WAIT_EXPIRED


class ListCall(C.Structure):
    """``bas_list_call`` of include/bas.h."""

    _fields_ = [("x_dev", C.c_void_p), ("ldx", C.c_int64), ("packed_dev", C.c_void_p), ("ids_dev", C.c_void_p),
                ("count_dev", C.c_void_p), ("bitmap_dev", C.c_void_p), ("y_dev", C.c_void_p), ("ldy", C.c_int64),
                ("k_host", C.c_int32), ("batch", C.c_int32), ("k", C.c_int32), ("n", C.c_int32),
                ("depends_on", C.c_int32), ("row_parallel", C.c_int32), ("op", C.c_int32), ("mask_entry", C.c_int32),
                ("mask_block0", C.c_int32), ("score_kind", C.c_int32), ("ids_out_dev", C.c_void_p),
                ("n_ids_dev", C.c_void_p), ("n_host", C.c_int32), ("shape_flags", C.c_int32)]


LIST_GEMM, LIST_SELECT = 0, 1
LIST_OUT_COMPACT, LIST_X_COMPACT, LIST_SELECT_SHARDED = 1, 2, 4


class StepCall(C.Structure):
    """``bas_step_call`` of include/bas.h."""

    _fields_ = [("w_host", C.c_void_p), ("n", C.c_int32), ("k", C.c_int32), ("batch", C.c_int32), ("n_keep", C.c_int32),
                ("score_kind", C.c_int32), ("reserved", C.c_int32)]


_PKG = Path(__file__).resolve().parent.parent
lib_path = _PKG / "libbas.so"


class BasError(RuntimeError):
    """A libbas entry point returned a non-zero status."""

    def __init__(self, status: int, where: str):
        self.status = int(status)
        msg = lib.bas_status_string(self.status).decode()
        extra = f" (cudaError {lib.bas_last_cuda_error()})" if self.status == 4 else ""
        super().__init__(f"{where}: {msg}{extra}")


def _load() -> C.CDLL:
    if not lib_path.exists():
        raise ImportError(
            f"{lib_path} is missing: build it with `python {_PKG.name}/build.py` "
            "(needs nvcc; there is no fallback implementation)")
    return C.CDLL(str(lib_path))


lib = _load()

_vp, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
_SIGNATURES = {
    "bas_status_string": (C.c_char_p, [_i]),
    "bas_last_cuda_error": (_i, []),
    "bas_launch_count": (C.c_ulonglong, []),
    "bas_set_wait_ms": (_i, [C.c_double]),
    "bas_packed_weight_bytes": (_sz, [_i, _i]),
    "bas_pack_weight": (_i, [_vp, _i, _i, _i64, _vp, _vp]),
    "bas_gemm_workspace_bytes": (_sz, [_i, _i]),
    "bas_workspace_init": (_i, [_vp, _sz, _vp]),
    "bas_gemm": (_i, [_vp, _i64, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _i64, _vp, _sz, _vp]),
    "bas_gemm_ex": (_i, [_vp, _i64, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _i64, _vp, _sz, _i, _vp]),
    "bas_read_device_status": (_i, [_vp, C.POINTER(C.c_uint), _vp]),
    "bas_build_bitmap": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "bas_select_workspace_bytes": (_sz, [_i]),
    "bas_select_topk": (_i, [_vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "bas_select_topk_weighted": (_i, [_vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "bas_select_budget": (_i, [_vp, _i64, _i, _i, C.c_double, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "bas_select_budget_ex": (_i, [_vp, _i64, _i, _i, C.c_double, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "bas_select_budget_capped": (_i, [_vp, _i64, _i, _i, C.c_double, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "bas_select_gemm": (_i, [_vp, _i64, _vp, _i, _i, _i, _i, _i, C.c_double, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _sz,
                             _vp, _sz, _i, _vp]),
    "bas_select_topk_noalloc": (_i, [_vp, _i64, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "bas_tp_create": (_i, [C.POINTER(_vp), _i, _i, _i, _i]),
    "bas_tp_handle": (_i, [_vp, _vp]),
    "bas_tp_connect": (_i, [_vp, _vp]),
    "bas_tp_disconnect": (_i, [_vp]),
    "bas_tp_destroy": (None, [_vp]),
    "bas_gemm_allreduce": (_i, [_vp, _vp, _i64, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _i64, _vp, _sz, _i, _vp]),
    "bas_list_create": (_i, [C.POINTER(_vp), _vp, _i, _i]),
    "bas_list_create_tp": (_i, [C.POINTER(_vp), _vp, _i, _i, _vp]),
    "bas_list_run": (_i, [_vp, _vp]),
    "bas_list_read_status": (_i, [_vp, C.POINTER(C.c_uint), _vp]),
    "bas_list_reset": (_i, [_vp]),
    "bas_list_set_wait": (_i, [_vp, C.c_double, _i]),
    "bas_list_info": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "bas_list_destroy": (None, [_vp]),
    "bas_step_create": (_i, [C.POINTER(_vp), _vp, _i, _i]),
    "bas_step_submit": (_i, [_vp, _vp, _vp, _vp]),
    "bas_step_wait": (_i, [_vp]),
    "bas_step_destroy": (None, [_vp]),
    "bas_linear_create": (_i, [C.POINTER(_vp), _vp, _i, _i, _i]),
    "bas_linear_forward_host": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "bas_linear_forward_host_ids": (_i, [_vp, _vp, _i, _vp, _i, _vp]),
    "bas_linear_submit_host": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "bas_linear_wait": (_i, [_vp]),
    "bas_linear_destroy": (None, [_vp]),
}
for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)       # AttributeError here = the library does not export the symbol
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTED = tuple(_SIGNATURES)


def check(status: int, where: str) -> None:
    if status != 0:
        raise BasError(status, where)


def launch_count() -> int:
    """Kernels launched by libbas from this process so far."""
    return int(lib.bas_launch_count())
