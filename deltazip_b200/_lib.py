"""ctypes binding of libdeltazip_b200.so (the C ABI declared in include/deltazip_b200.h).

The library must be present: there is no CPU or PyTorch fallback for any of
its entry points.  Build it with `python -m deltazip_b200.build`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libdeltazip_b200.so")

DZ_OK = 0
DZ_ERR_INVALID_ARG = 1
DZ_ERR_SHAPE = 2
DZ_ERR_ALIGNMENT = 3
DZ_ERR_WORKSPACE = 4
DZ_ERR_SLOT_RANGE = 5
DZ_ERR_NOT_2_4 = 6
DZ_ERR_NOT_SYMMETRIC = 7
DZ_ERR_CUDA = 8
DZ_ERR_TIMEOUT = 9
DZ_ERR_UNSUPPORTED = 10
DZ_ERR_TOO_LARGE = 11

DZ_DTYPE_F16 = 0
DZ_DTYPE_BF16 = 1
DZ_DTYPE_F32 = 2
DZ_INDEX_I32 = 0
DZ_INDEX_I64 = 1
DZ_SBMM_ACCUMULATE = 1
DZ_SBMM_INPUTS_STABLE = 2


class PushTarget(Structure):
    """Mirror of dz_push_target."""
    _fields_ = [("world", c_int32), ("rank", c_int32), ("epoch", c_uint32), ("reserved", c_uint32),
                ("data", c_void_p * 8), ("flags", c_void_p * 8)]


class SbmmArgs(Structure):
    """Mirror of dz_sbmm_args."""
    _fields_ = [
        ("x", c_void_p), ("w_base", c_void_p),
        ("qweight", c_void_p), ("meta", c_void_p), ("scales", c_void_p),
        ("qweight_stride", c_int64), ("meta_stride", c_int64), ("scales_stride", c_int64),
        ("segments", c_void_p), ("y", c_void_p),
        ("M", c_int32), ("N", c_int32), ("K", c_int32),
        ("num_slots", c_int32), ("bits", c_int32), ("dtype", c_int32),
        ("tokens_sorted", c_int32), ("flags", c_int32),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("y_stride", c_int64),
        ("push", POINTER(PushTarget)),
    ]


class DeltaZipError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        msg = f"{where}: {status_string(status)} (dz_status {status})"
        if detail:
            msg += f" [{detail}]"
        super().__init__(msg)


_lib = None

_SIGNATURES = {
    "dz_version": (c_int, []),
    "dz_status_string": (c_char_p, [c_int]),
    "dz_last_cuda_error": (c_char_p, []),
    "dz_slot_qweight_bytes": (c_size_t, [c_int, c_int, c_int]),
    "dz_slot_meta_bytes": (c_size_t, [c_int, c_int]),
    "dz_slot_scales_bytes": (c_size_t, [c_int]),
    "dz_convert_from_gptq": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "dz_unpack": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "dz_segments_bytes": (c_size_t, [c_int, c_int]),
    "dz_build_segments": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "dz_sbmm_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "dz_sbmm": (c_int, [POINTER(SbmmArgs), c_void_p]),
    "dz_base_gemm": (c_int, [POINTER(SbmmArgs), c_void_p]),
    "dz_sbmm_static": (c_int, [POINTER(SbmmArgs), c_void_p]),
    "dz_sbmm_static_max_tokens": (c_int, []),
    "dz_sbmm_static_status": (c_int, [c_void_p, POINTER(c_int)]),
    "dz_delta_embedding": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p]),
    "dz_grouped_gemm_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "dz_grouped_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_int64, c_void_p, c_size_t, c_void_p]),
    "dz_quant_find_params": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "dz_sparsegpt_block": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "dz_pack_gptq": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p]),
    "dz_rms_norm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]),
    "dz_silu_and_mul": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "dz_rotary_and_cache": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                    c_int, c_int, c_float, c_int, c_void_p]),
    "dz_paged_attention_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "dz_paged_attention_decode": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                          c_void_p, c_size_t, c_int, c_void_p]),
    "dz_slot_upload": (c_int, [c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "dz_slot_reset": (c_int, [c_void_p, c_size_t, c_void_p]),
    "dz_stream_fence": (c_int, [c_void_p]),
    "dz_read_status": (c_int, [c_void_p, c_void_p, POINTER(c_int)]),
    "dz_allreduce_region_bytes": (c_size_t, [c_size_t]),
    "dz_allreduce_create": (c_int, [POINTER(c_void_p), c_int, c_int, c_size_t]),
    "dz_allreduce_create_external": (c_int, [POINTER(c_void_p), c_int, c_int, c_size_t, POINTER(c_void_p), c_void_p]),
    "dz_allreduce_export": (c_int, [c_void_p, c_void_p]),
    "dz_allreduce_connect": (c_int, [c_void_p, c_void_p]),
    "dz_allreduce_staging": (c_int, [c_void_p, POINTER(c_void_p), POINTER(c_size_t)]),
    "dz_allreduce_run": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "dz_allreduce_status": (c_int, [c_void_p, POINTER(c_int)]),
    "dz_allreduce_set_variant": (c_int, [c_void_p, c_int]),
    "dz_allreduce_push_target": (c_int, [c_void_p, c_int, c_int, c_int, POINTER(PushTarget)]),
    "dz_allreduce_run_pushed": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "dz_allreduce_destroy": (c_int, [c_void_p]),
}


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m deltazip_b200.build` "
                "(there is no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = argtypes
        for name in ("dz_sbmm_simt",):  # validation twins, not part of the public header
            if hasattr(handle, name):
                fn = getattr(handle, name)
                fn.restype = c_int
                fn.argtypes = [POINTER(SbmmArgs), c_void_p]
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().dz_status_string(int(status)).decode()


def check(status: int, where: str) -> None:
    if status != DZ_OK:
        detail = lib().dz_last_cuda_error().decode() if status == DZ_ERR_CUDA else ""
        raise DeltaZipError(status, where, detail)
