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


def _args(layer, x, seg, y, ws=None, base=True):
    from deltazip_b200 import _lib
    return _lib.SbmmArgs(
        x=x.data_ptr(), w_base=layer.w.data_ptr() if base else None, qweight=layer.qweight.data_ptr(),
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
        a = _args(layer, x, seg, y)
        _lib.check(L.dz_sbmm_static(ctypes.byref(a), stream), "dz_sbmm_static")
        torch.cuda.synchronize()
        assert torch.equal(y, y_ref), f"call {call}: static-scratch output differs from dz_sbmm"
        assert O.rel_l2(y.cpu().numpy(), layer.oracle(x_np, idx_np)) <= 1e-2
        # a further call changes nothing about the device's memory: the driver reports the same
        # free byte count before and after (nothing was allocated or freed on its behalf)
        free0, _ = torch.cuda.mem_get_info()
        _lib.check(L.dz_sbmm_static(ctypes.byref(a), stream), "dz_sbmm_static")
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert free0 == free1
        assert torch.equal(y, y_ref)
        # delta-only form (no base weight), as dz_sbmm accepts it
        y_only_ref = torch.empty_like(y_ref)
        _lib.check(L.dz_sbmm(ctypes.byref(_args(layer, x, seg, y_only_ref, ws, base=False)), stream),
                   "dz_sbmm")
        y_only = torch.full_like(y, float("nan"))
        _lib.check(L.dz_sbmm_static(ctypes.byref(_args(layer, x, seg, y_only, base=False)), stream),
                   "dz_sbmm_static")
        torch.cuda.synchronize()
        assert torch.equal(y_only, y_only_ref)
        host = ctypes.c_int(-1)
        _lib.check(L.dz_sbmm_static_status(stream, ctypes.byref(host)), "dz_sbmm_static_status")
        assert host.value == 0


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


def test_static_scratch_status_word_is_readable_and_sticky():
    """A batch the kernel rejects on the device (the caller promised sorted tokens, the table
    says otherwise) computes nothing; the finding stays in the built-in scratch across later
    calls until dz_sbmm_static_status reads and clears it.  The kernel returns normally: no
    fault is involved."""
    from deltazip_b200 import _lib, ops
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    layer = DeviceLayer(256, 256, 3, 4, seed=8)
    x_np, idx_np = O.make_tokens(24, 256, 3, seed=8, sort=False)
    assert (np.diff(idx_np) < 0).any()
    x = dev(x_np)
    seg = ops.Segments(24, 3, "cuda").build(dev(idx_np))          # table records "not sorted"
    y = torch.full((24, 256), 7.0, dtype=torch.float16, device="cuda")
    a = _args(layer, x, seg, y)                                   # ... but the call promises sorted
    host = ctypes.c_int(-1)
    _lib.check(L.dz_sbmm_static_status(stream, ctypes.byref(host)), "dz_sbmm_static_status")
    _lib.check(L.dz_sbmm_static(ctypes.byref(a), stream), "dz_sbmm_static")
    torch.cuda.synchronize()
    assert (y == 7.0).all()                                       # nothing was computed
    # a correct call in between does not clear the word
    xs_np, idxs_np = O.make_tokens(24, 256, 3, seed=9)
    seg2 = ops.Segments(24, 3, "cuda").build(dev(idxs_np), sorted_hint=True)
    y2 = torch.empty((24, 256), dtype=torch.float16, device="cuda")
    _lib.check(L.dz_sbmm_static(ctypes.byref(_args(layer, dev(xs_np), seg2, y2)), stream), "dz_sbmm_static")
    _lib.check(L.dz_sbmm_static_status(stream, ctypes.byref(host)), "dz_sbmm_static_status")
    assert host.value == _lib.DZ_ERR_INVALID_ARG
    assert O.rel_l2(y2.cpu().numpy(), layer.oracle(xs_np, idxs_np)) <= 1e-2
    _lib.check(L.dz_sbmm_static_status(stream, ctypes.byref(host)), "dz_sbmm_static_status")
    assert host.value == 0                                        # cleared by the read
