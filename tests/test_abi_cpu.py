"""CPU-side checks of the C-ABI library: it builds, loads, exports every symbol
the public header declares, and its pure host functions answer (no GPU work)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def handle():
    from deltazip_b200 import build
    path = build.build_library()
    return ctypes.CDLL(path)


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "deltazip_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dz_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for must in ("dz_sbmm", "dz_base_gemm", "dz_convert_from_gptq", "dz_unpack",
                 "dz_build_segments", "dz_slot_upload"):
        assert must in names


def test_every_declared_symbol_is_exported(handle):
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"


def test_host_functions(handle):
    from deltazip_b200 import _lib
    L = _lib.lib()
    assert L.dz_version() >= 100
    assert L.dz_slot_qweight_bytes(4096, 4096, 4) == 4096 * 4096 // 4
    assert L.dz_slot_qweight_bytes(4096, 4096, 2) == 4096 * 4096 // 8
    assert L.dz_slot_meta_bytes(4096, 4096) == 4096 * 4096 // 8
    assert L.dz_slot_qweight_bytes(100, 4096, 4) == 0      # N % 128 != 0
    assert L.dz_slot_qweight_bytes(128, 4096, 3) == 0      # 3-bit unsupported
    assert L.dz_segments_bytes(64, 8) > 64
    assert L.dz_sbmm_workspace_bytes(64, 4096, 4096, 1) > 0
    assert L.dz_sbmm_workspace_bytes(64, 4096, 4096, 0) > L.dz_sbmm_workspace_bytes(64, 4096, 4096, 1)
    assert b"2:4" in L.dz_status_string(_lib.DZ_ERR_NOT_2_4)


def test_argument_validation_without_gpu(handle):
    """Invalid arguments are rejected before any CUDA call is made."""
    from deltazip_b200 import _lib
    L = _lib.lib()
    assert L.dz_sbmm(None, None) == _lib.DZ_ERR_INVALID_ARG
    a = _lib.SbmmArgs(x=16, w_base=16, y=16, M=4, N=100, K=64, bits=4, num_slots=1)
    assert L.dz_sbmm(ctypes.byref(a), None) == _lib.DZ_ERR_SHAPE
    a = _lib.SbmmArgs(x=8, w_base=16, y=16, M=4, N=128, K=64, bits=4, num_slots=1)
    assert L.dz_sbmm(ctypes.byref(a), None) == _lib.DZ_ERR_ALIGNMENT
    a = _lib.SbmmArgs(x=16, w_base=16, y=16, M=4, N=128, K=64, bits=4, num_slots=1, dtype=7)
    assert L.dz_sbmm(ctypes.byref(a), None) == _lib.DZ_ERR_INVALID_ARG      # unknown dtype
    assert L.dz_build_segments(None, 0, 4, 2, None, None) == _lib.DZ_ERR_INVALID_ARG
    assert L.dz_convert_from_gptq(None, None, None, 128, 64, 4, None, None, None, None, None) \
        == _lib.DZ_ERR_INVALID_ARG


def test_ops_refuse_cpu_tensors():
    import torch
    from deltazip_b200 import ops
    x = torch.zeros(4, 64, dtype=torch.float16)
    with pytest.raises(ValueError):
        ops.base_gemm(x, torch.zeros(128, 64, dtype=torch.float16))
