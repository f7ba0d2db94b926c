"""ctypes binding of ``liblf_b200.so`` (declared in ``include/liteform_b200.h``).

There is no CPU or PyTorch fallback behind these calls: if the shared library has not been
built, or a call reports an error, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

from . import _build
from ._build import LIB_PATH

LF_OK = 0
LF_ERR_INVALID_ARGUMENT = -1
LF_ERR_CUDA = -2
LF_ERR_WORKSPACE_TOO_SMALL = -3
LF_ERR_UNSUPPORTED = -4
LF_ERR_KERNEL_TIMEOUT = -5

LF_OPT_SPMM_SLOTS_PER_GROUP = 1
LF_OPT_SPMM_CACHE_POLICY = 2
LF_OPT_SPMM_MIN_BLOCKS = 3
LF_OPT_BSR_COPY_ENGINE = 4
LF_OPT_BSR_TILE_ORDER = 5
LF_OPT_SPMM_TILE_SEGMENTS = 6
LF_OPT_BSR_PIPE_SHAPE = 7
LF_OPT_BSR_PIPE_3D = 8
LF_OPT_BSR_UMMA_PRODUCER = 9
LF_OPT_SPMM_GATHER_RING = 10
LF_OPT_BSR_BLOCK_WARPS = 11
LF_OPT_SPMM_RING_MIN_SLOTS = 12
LF_DTYPE_F32, LF_DTYPE_BF16, LF_DTYPE_F16 = 0, 1, 2
LF_SPMM_OVERWRITE = 0
LF_SPMM_ACCUMULATE = 1
LF_SPMM_NO_SYNC = 2
LF_SPMM_FORMAT_RESIDENT = 4
NUM_WIDTH_CLASSES = 11
COLMASK_BINS = 2048
STATIC_STATS_MAX_COLS = 1 << 20

i32p = C.POINTER(C.c_int32)
i64p = C.POINTER(C.c_int64)
f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)
vp = C.c_void_p


class LfHyb(C.Structure):
    """Mirror of ``struct lf_hyb``."""
    _fields_ = [
        ("num_rows", C.c_int64), ("num_cols", C.c_int64),
        ("row_begin", C.c_int64), ("row_end", C.c_int64),
        ("num_parts", C.c_int32), ("num_buckets", C.c_int32),
        ("part_bucket_off", vp), ("widths", vp), ("ell_rows", vp), ("row_off", vp), ("slot_off", vp),
        ("rows", vp), ("cols", vp), ("vals", vp), ("mask", vp), ("zero_rows", vp),
        ("num_zero_rows", C.c_int64),
    ]


class LiteformError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"liteform_b200 error {status}: {message}")
        self.status = status
        self.message = message


# every exported symbol with (restype, argtypes); tests check that the library exports them all
SIGNATURES = {
    "lf_version": (C.c_int, []),
    "lf_last_error": (C.c_char_p, []),
    "lf_set_option": (C.c_int, [C.c_int32, C.c_int32]),
    "lf_csr_validate": (C.c_int, [vp, vp, C.c_int64, C.c_int64, C.c_int64, vp]),
    "lf_hyb_stats_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int32]),
    "lf_hyb_stats": (C.c_int, [vp, vp, C.c_int64, C.c_int64, C.c_int32, vp, vp, vp, C.c_size_t, vp]),
    "lf_hyb_stats_static": (C.c_int, [vp, vp, C.c_int64, C.c_int64, C.c_int32, vp, vp, vp]),
    "lf_hyb_build_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int32, C.c_int32]),
    "lf_hyb_fill_scratch_bytes": (C.c_size_t, [C.c_int64]),
    "lf_hyb_plan": (C.c_int, [vp, vp, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int32, vp, vp,
                              vp, vp, vp, vp, vp, C.c_size_t, vp]),
    "lf_hyb_fill": (C.c_int, [vp, vp, vp, C.POINTER(LfHyb), vp, C.c_size_t, vp, C.c_size_t, vp]),
    "lf_spmm_hyb_f32_kernel_name": (C.c_char_p, [C.POINTER(LfHyb), vp, C.c_int64, vp, C.c_int64, C.c_int32]),
    "lf_spmm_hyb_f32": (C.c_int, [C.POINTER(LfHyb), vp, C.c_int64, vp, C.c_int64, C.c_int32, C.c_int32, vp]),
    "lf_spmm_hyb_bf16": (C.c_int, [C.POINTER(LfHyb), vp, C.c_int64, vp, C.c_int64, C.c_int32, C.c_int32, vp]),
    "lf_spmm_hyb_f32_bcast": (C.c_int, [C.POINTER(LfHyb), vp, C.c_int64, vp, C.c_int32, C.c_int64, C.c_int32, vp]),
    "lf_allgather_rows": (C.c_int, [vp, C.c_int64, C.c_int64, C.c_int64, C.c_int32, vp, C.c_int32, C.c_int64, vp]),
    "lf_spmm_hyb_f32_host_workspace_bytes": (C.c_size_t, [C.POINTER(LfHyb), C.c_int32]),
    "lf_spmm_hyb_f32_host": (C.c_int, [C.POINTER(LfHyb), vp, vp, C.c_int32, C.c_int32, vp, C.c_size_t, vp]),
    "lf_spmm_csr_f32": (C.c_int, [vp, vp, vp, C.c_int64, C.c_int64, C.c_int64, vp, C.c_int64, vp, C.c_int64, C.c_int32, vp]),
    "lf_bsr8_plan": (C.c_int, [vp, vp, C.c_int64, vp, C.POINTER(C.c_int64), vp]),
    "lf_bsr8_fill": (C.c_int, [vp, vp, vp, C.c_int64, vp, vp, vp, C.c_int32, vp]),
    "lf_bsr_split8_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int32, C.c_int32]),
    "lf_bsr_split8_plan": (C.c_int, [vp, vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_int32, vp, C.c_size_t, vp,
                                     C.POINTER(C.c_int64), vp]),
    "lf_bsr_split8_fill": (C.c_int, [vp, vp, vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, C.c_int32, vp, vp, vp, vp,
                                     C.c_int32, vp]),
    "lf_bsr_set_tuning": (C.c_int, [C.c_int32, C.c_int32, C.c_int32]),
    "lf_bsr_copy_status": (C.c_int, [vp]),
    "lf_spmm_bsr8_f32": (C.c_int, [vp, vp, vp, C.c_int64, C.c_int64, vp, C.c_int64, vp, C.c_int64, C.c_int32, vp]),
    "lf_spmm_bsr8_bf16": (C.c_int, [vp, vp, vp, C.c_int64, C.c_int64, vp, C.c_int64, vp, C.c_int64, C.c_int32, vp]),
    "lf_spmm_bsr8_f16": (C.c_int, [vp, vp, vp, C.c_int64, C.c_int64, vp, C.c_int64, vp, C.c_int64, C.c_int32, vp]),
    "lf_row_stats_blocks": (C.c_int64, [C.c_int64, C.c_int64]),
    "lf_row_stats": (C.c_int, [vp, C.c_int64, C.c_int64, vp, vp]),
    "lf_shard_rows": (C.c_int, [vp, C.c_int64, C.c_int32, vp, vp]),
}

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m liteform_ae_b200._build` "
                "(there is no fallback implementation)")
        if _build.is_stale():
            raise RuntimeError(
                f"{LIB_PATH} is older than its sources: rebuild it with `python -m liteform_ae_b200._build` "
                "(a stale library is an error, not a fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != LF_OK:
        msg = load().lf_last_error()
        raise LiteformError(status, msg.decode("utf-8", "replace") if msg else "")


def np_ptr(arr) -> int:
    """Address of a C-contiguous NumPy array (0 for None)."""
    if arr is None:
        return 0
    assert arr.flags["C_CONTIGUOUS"]
    return arr.ctypes.data


def t_ptr(tensor) -> int:
    """Address of a contiguous torch tensor (0 for None)."""
    if tensor is None:
        return 0
    assert tensor.is_contiguous()
    return tensor.data_ptr()
