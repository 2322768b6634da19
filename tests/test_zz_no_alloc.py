"""dz_sbmm_static: the SBMM entry point that allocates nothing.

Meant for hosts that may not call cudaMalloc where they call this library (all
device memory already given to their own pool, or an allocator they must not
touch): the kernel's scratch is a fixed array inside the library instead of a
caller-provided workspace.  The test calls it through the C ABI, twice in a row
(the array is shared and keeps the previous call's contents), and requires the
same output as dz_sbmm on the same inputs -- bit for bit, since both run the
same kernel with the same work split.  This file sorts last so that a run that
stops at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import deltazip_oracle as O
from tests.gpu_util import DeviceLayer, dev

pytestmark = pytest.mark.gpu


def _args(layer, x, seg, y, ws=None):
    from deltazip_b200 import _lib
    return _lib.SbmmArgs(
        x=x.data_ptr(), w_base=layer.w.data_ptr(), qweight=layer.qweight.data_ptr(),
        meta=layer.meta.data_ptr(), scales=layer.scales.data_ptr(),
        qweight_stride=layer.qweight.stride(0) * 4, meta_stride=layer.meta.stride(0) * 2,
        scales_stride=layer.scales.stride(0) * 2, segments=seg.buf.data_ptr(), y=y.data_ptr(),
        M=x.shape[0], N=layer.n, K=layer.k, num_slots=layer.num_slots, bits=layer.bits,
        dtype=_lib.DZ_DTYPE_F16, tokens_sorted=1,
        workspace=ws.data_ptr() if ws is not None else None,
        workspace_bytes=ws.numel() if ws is not None else 0)


def test_static_scratch_entry_matches_dz_sbmm_twice():
    from deltazip_b200 import _lib, ops
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert L.dz_sbmm_static_max_tokens() == 64
    for call, (n, k, m, nd, bits) in enumerate([(1024, 2048, 64, 8, 4), (512, 1728, 37, 5, 2)]):
        layer = DeviceLayer(n, k, nd, bits, seed=40 + call)
        x_np, idx_np = O.make_tokens(m, k, nd, seed=40 + call)
        x = dev(x_np)
        seg = ops.Segments(m, nd, "cuda").build(dev(idx_np), sorted_hint=True)
        # existing entry point, caller-provided workspace
        ws = torch.zeros(L.dz_sbmm_workspace_bytes(m, n, k, 1), dtype=torch.uint8, device="cuda")
        y_ref = torch.empty((m, n), dtype=torch.float16, device="cuda")
        _lib.check(L.dz_sbmm(ctypes.byref(_args(layer, x, seg, y_ref, ws)), stream), "dz_sbmm")
        # new entry point: no workspace at all
        y = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        _lib.check(L.dz_sbmm_static(ctypes.byref(_args(layer, x, seg, y)), stream), "dz_sbmm_static")
        torch.cuda.synchronize()
        assert torch.equal(y, y_ref), f"call {call}: static-scratch output differs from dz_sbmm"
        assert O.rel_l2(y.cpu().numpy(), layer.oracle(x_np, idx_np)) <= 1e-2


def test_static_scratch_entry_rejects_what_does_not_fit():
    from deltazip_b200 import _lib, ops
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    layer = DeviceLayer(128, 128, 2, 4, seed=3)
    m = 65                                            # one token more than the scratch is sized for
    x_np, idx_np = O.make_tokens(m, 128, 2, seed=3)
    x = dev(x_np)
    seg = ops.Segments(m, 2, "cuda").build(dev(idx_np), sorted_hint=True)
    y = torch.empty((m, 128), dtype=torch.float16, device="cuda")
    a = _args(layer, x, seg, y)
    assert L.dz_sbmm_static(ctypes.byref(a), stream) == _lib.DZ_ERR_TOO_LARGE
    a.M = 8
    a.tokens_sorted = 0                               # the unsorted path needs a gather buffer
    assert L.dz_sbmm_static(ctypes.byref(a), stream) == _lib.DZ_ERR_TOO_LARGE
