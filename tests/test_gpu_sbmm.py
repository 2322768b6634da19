"""GPU parity of the SBMM hot path, called through the C ABI (ctypes).

Tolerance: layer outputs within rel-L2 <= 1e-2 of the reference path in fp16
(the bar the task states); in practice the fused fp32 accumulation lands near
1e-3 of the oracle's fp16 result and closer still to the fp32 "true" value.
"""
import numpy as np
import pytest
import torch

from oracle import deltazip_oracle as O
from tests.gpu_util import DeviceLayer, dev

pytestmark = pytest.mark.gpu
TOL = 1e-2


def run_sbmm(layer, x_np, idx_np, entry="dz_sbmm", index_dtype=torch.int64):
    from deltazip_b200 import ops
    x = dev(x_np)
    idx = torch.from_numpy(np.asarray(idx_np)).to(index_dtype).cuda()
    # the host knows the order here, as a scheduler would: promise "sorted" when it is, so that
    # both the in-place path and the gather path are exercised
    c = np.where((np.asarray(idx_np) >= layer.num_slots) | (np.asarray(idx_np) < -1), -1, idx_np)
    hint = bool(len(c) < 2 or (np.diff(c) >= 0).all())
    seg = ops.Segments(max(len(idx_np), 1), layer.num_slots, "cuda").build(idx, sorted_hint=hint)
    y = ops.sbmm(x, layer.qweight, layer.scales, layer.meta, seg, layer.w, _entry=entry)
    torch.cuda.synchronize()
    return y.cpu().numpy(), seg


def check(layer, x_np, idx_np, y):
    ref = layer.oracle(x_np, idx_np)
    assert y.shape == ref.shape
    assert np.isfinite(y.astype(np.float32)).all()
    err = O.rel_l2(y, ref)
    assert err <= TOL, f"rel-L2 {err}"
    # per-token check: no single row may hide behind the batch norm
    for i in range(len(idx_np)):
        assert O.rel_l2(y[i], ref[i]) <= 2 * TOL, f"row {i} slot {idx_np[i]}"
    true = layer.oracle_fp32(x_np, idx_np)
    assert O.rel_l2(y, true) <= 2e-3


@pytest.mark.parametrize("entry", ["dz_sbmm", "dz_sbmm_simt"])
@pytest.mark.parametrize("bits", [4, 2])
def test_config1_shape_small(entry, bits):
    """One delta, 16 tokens (the shape of the single-layer config, at 1024x1024)."""
    layer = DeviceLayer(1024, 1024, 1, bits, seed=0)
    x, idx = O.make_tokens(16, 1024, 1, seed=0)
    y, _ = run_sbmm(layer, x, idx, entry)
    check(layer, x, idx, y)


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("n,k,m,nd", [(256, 512, 64, 8), (384, 448, 37, 5), (128, 64, 1, 1),
                                      (512, 1728, 100, 16), (1024, 256, 300, 3)])
def test_shapes_sorted(bits, n, k, m, nd):
    layer = DeviceLayer(n, k, nd, bits, seed=n + m)
    x, idx = O.make_tokens(m, k, nd, seed=m, base_frac=0.1)
    y, seg = run_sbmm(layer, x, idx)
    hdr = seg.header()
    assert hdr[0] == m and hdr[3] == 1 and hdr[4] == 0
    check(layer, x, idx, y)


@pytest.mark.parametrize("index_dtype", [torch.int64, torch.int32])
def test_unsorted_tokens(index_dtype):
    layer = DeviceLayer(256, 256, 6, 4, seed=7, num_slots=8)
    x, idx = O.make_tokens(90, 256, 6, seed=3, sort=False, base_frac=0.2)
    y, seg = run_sbmm(layer, x, idx, index_dtype=index_dtype)
    assert seg.header()[3] == 0
    check(layer, x, idx, y)


def test_all_base_tokens_and_base_gemm():
    from deltazip_b200 import ops
    layer = DeviceLayer(256, 320, 2, 4, seed=9)
    x, _ = O.make_tokens(33, 320, 2, seed=1)
    idx = np.full(33, -1, dtype=np.int64)
    y, _ = run_sbmm(layer, x, idx)
    ref = O.base_linear(x, layer.w_np)
    assert O.rel_l2(y, ref) <= 2e-3
    y2 = ops.base_gemm(dev(x), layer.w).cpu().numpy()
    np.testing.assert_array_equal(y2.view(np.uint16), y.view(np.uint16))


def test_out_of_range_slot_is_reported_and_treated_as_base():
    from deltazip_b200 import _lib
    layer = DeviceLayer(128, 128, 2, 4, seed=2)
    x, idx = O.make_tokens(8, 128, 2, seed=2)
    idx = idx.copy()
    idx[-1] = 5
    y, seg = run_sbmm(layer, x, idx)
    assert seg.header()[4] == _lib.DZ_ERR_SLOT_RANGE
    idx_ref = idx.copy()
    idx_ref[-1] = -1
    check(layer, x, idx_ref, y)


def test_empty_batch():
    from deltazip_b200 import ops
    layer = DeviceLayer(128, 64, 1, 4, seed=1)
    x = torch.zeros((0, 64), dtype=torch.float16, device="cuda")
    seg = ops.Segments(1, 1, "cuda").build(torch.zeros(0, dtype=torch.int64, device="cuda"))
    y = ops.sbmm(x, layer.qweight, layer.scales, layer.meta, seg, layer.w)
    assert y.shape == (0, 128)


def test_apply_delta_reference_signature():
    """The op keeps the reference's argument order and semantics."""
    from deltazip_b200 import ops
    layer = DeviceLayer(256, 256, 4, 4, seed=11)
    x, idx = O.make_tokens(24, 256, 4, seed=5)
    y = ops.apply_delta(dev(x), layer.qweight, layer.scales, layer.meta, dev(idx), layer.w)
    check(layer, x, idx, y.cpu().numpy())


def test_linearity_property_full_size():
    """Size-independent property at a benchmark shape (4096x4096, 8 deltas, 64
    tokens): f(2x) == 2 f(x) exactly in fp16 (power-of-two scaling commutes with
    every rounding while nothing overflows), and tokens that share a slot and
    an input row produce identical outputs whatever their position."""
    from deltazip_b200 import ops
    layer = DeviceLayer(4096, 4096, 8, 4, seed=21)
    x, idx = O.make_tokens(64, 4096, 8, seed=21)
    x[1] = x[0]
    idx[:2] = idx[0]
    seg = ops.Segments(64, 8, "cuda").build(dev(idx))
    y1 = ops.sbmm(dev(x), layer.qweight, layer.scales, layer.meta, seg, layer.w).cpu().numpy()
    y2 = ops.sbmm(dev(x * np.float16(2)), layer.qweight, layer.scales, layer.meta, seg, layer.w).cpu().numpy()
    # exact wherever the result is a normal fp16 number (a subnormal result has
    # fewer significant bits than its double, so rounding may differ there)
    normal = np.abs(y1.astype(np.float32)) >= 2.0 ** -13
    assert normal.mean() > 0.999
    np.testing.assert_array_equal((y1 * np.float16(2)).view(np.uint16)[normal],
                                  y2.view(np.uint16)[normal])
    np.testing.assert_array_equal(y1[0].view(np.uint16), y1[1].view(np.uint16))
    # spot-check 4 rows against the oracle at full size
    rows = [0, 17, 40, 63]
    ref = layer.oracle(x[rows], idx[rows])
    assert O.rel_l2(y1[rows], ref) <= TOL


def test_deterministic_across_runs():
    from deltazip_b200 import ops
    layer = DeviceLayer(512, 2048, 8, 4, seed=4)
    x, idx = O.make_tokens(64, 2048, 8, seed=4)
    seg = ops.Segments(64, 8, "cuda").build(dev(idx))
    xd = dev(x)
    y0 = ops.sbmm(xd, layer.qweight, layer.scales, layer.meta, seg, layer.w).clone()
    for _ in range(5):
        y = ops.sbmm(xd, layer.qweight, layer.scales, layer.meta, seg, layer.w)
        assert torch.equal(y, y0)


@pytest.mark.parametrize("bits", [4, 2])
def test_bf16_activations_and_base(bits):
    """bf16 base weights / activations (scales stay fp16, as in the reference's layers,
    serving/vllm/delta/layers_marlin.py:319-325).  Reference: the same formula in float32 on
    the bf16 values; tolerance rel-L2 <= 1e-2 (bf16 keeps 8 significant bits)."""
    from deltazip_b200 import ops
    layer = DeviceLayer(512, 1024, 6, bits, seed=31)
    x_np, idx_np = O.make_tokens(75, 1024, 6, seed=31, base_frac=0.15)
    xb = dev(x_np).to(torch.bfloat16)
    wb = layer.w.to(torch.bfloat16)
    seg = ops.Segments(75, 6, "cuda").build(dev(idx_np))
    y = ops.sbmm(xb, layer.qweight, layer.scales, layer.meta, seg, wb)
    assert y.dtype == torch.bfloat16
    ref = xb.float() @ wb.float().t()
    dense = [torch.from_numpy(d).cuda().float() for d in layer.dense()]
    idx = torch.from_numpy(idx_np).cuda()
    for d in range(6):
        rows = idx == d
        ref[rows] += xb[rows].float() @ dense[d].t()
    err = O.rel_l2(y.float().cpu().numpy(), ref.cpu().numpy())
    assert err <= TOL, err
    assert ops.read_status() == 0
    yb = ops.base_gemm(xb, wb)
    assert O.rel_l2(yb.float().cpu().numpy(), (xb.float() @ wb.float().t()).cpu().numpy()) <= 5e-3


@pytest.mark.parametrize("bits", [4, 2])
def test_add_delta_in_place_matches_the_separate_base_output_path(bits):
    """The GPTQ-layout form of the op (base output first, delta added in place,
    serving/vllm/delta/deltazip.py:14-38): y = fp16(x W^T) + delta products."""
    from deltazip_b200 import ops
    layer = DeviceLayer(384, 512, 5, bits, seed=21)
    x, idx = O.make_tokens(40, 512, 5, seed=9)
    xd, idxd = dev(x), dev(idx)
    # delta products alone (no base weight): rows of slot -1 are exactly zero
    seg = ops.Segments(len(idx), layer.num_slots, "cuda").build(idxd)
    only = ops.sbmm(xd, layer.qweight, layer.scales, layer.meta, seg, None)
    dense = layer.dense()
    want = np.zeros((len(idx), 384), np.float32)
    for i, s in enumerate(idx):
        if s >= 0:
            want[i] = x[i].astype(np.float32) @ dense[s].astype(np.float32).T
    torch.cuda.synchronize()
    got = only.float().cpu().numpy()
    assert O.rel_l2(got, want) <= 2e-3
    assert not got[np.asarray(idx) < 0].any()
    # in place on top of a base output
    y = ops.base_gemm(xd, layer.w)
    base = y.clone()
    ret = ops.add_delta(y, xd, layer.qweight, None, layer.scales, None, idxd, meta=layer.meta)
    assert ret.data_ptr() == y.data_ptr()
    torch.cuda.synchronize()
    # the kernel adds in fp32 and rounds once; base + fp16(delta products) rounds twice
    two_step = (base.float() + only.float()).cpu().numpy()
    assert O.rel_l2(y.float().cpu().numpy(), two_step) <= 1e-3
    check(layer, x, idx, y.cpu().numpy())


def test_apply_delta_packed_nslice_merged_layer():
    """Three sub-layers with their own stacks written into slices of one output."""
    from deltazip_b200 import ops
    widths = (256, 128, 128)
    layers_ = [DeviceLayer(w, 256, 3, 4, seed=30 + i) for i, w in enumerate(widths)]
    x, idx = O.make_tokens(20, 256, 3, seed=4)
    xd, idxd = dev(x), dev(idx)
    out = torch.cat([ops.base_gemm(xd, l.w) for l in layers_], dim=1)
    ops.apply_delta_packed_nslice(xd, [l.qweight for l in layers_], None, [l.scales for l in layers_],
                                  None, idxd, out, widths, meta_stacked=[l.meta for l in layers_])
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    off = 0
    for l, w in zip(layers_, widths):
        check(l, x, idx, got[:, off:off + w])
        off += w


def test_apply_delta_sees_new_and_rewritten_index_tensors():
    """The drop-in op caches the segment table per index tensor.  A new tensor (even one the
    allocator places at the address of a freed one) and an in-place rewrite of the same tensor
    (what the reference's _set_delta_mapping does with copy_) must both rebuild the table."""
    from deltazip_b200 import ops
    layer = DeviceLayer(256, 256, 4, 4, seed=12)
    x, idx_a = O.make_tokens(32, 256, 4, seed=6)
    _, idx_b = O.make_tokens(32, 256, 4, seed=7)
    assert (idx_a != idx_b).any()
    xd = dev(x)
    ia = dev(idx_a)
    ya = ops.apply_delta(xd, layer.qweight, layer.scales, layer.meta, ia, layer.w).cpu().numpy()
    check(layer, x, idx_a, ya)
    del ia
    ib = dev(idx_b)                       # may reuse the freed tensor's address
    yb = ops.apply_delta(xd, layer.qweight, layer.scales, layer.meta, ib, layer.w).cpu().numpy()
    check(layer, x, idx_b, yb)
    ib.copy_(dev(idx_a))                  # same tensor, new contents
    yc = ops.apply_delta(xd, layer.qweight, layer.scales, layer.meta, ib, layer.w).cpu().numpy()
    check(layer, x, idx_a, yc)
    # repeated calls on an unchanged tensor reuse the table and agree bit for bit
    yd = ops.apply_delta(xd, layer.qweight, layer.scales, layer.meta, ib, layer.w).cpu().numpy()
    np.testing.assert_array_equal(yc.view(np.uint16), yd.view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 4])
def test_prefill_sized_batch_takes_the_split_path_and_agrees_with_the_fused_one(bits):
    """More than ops.FUSED_MAX_TOKENS rows: dense product through the library GEMM, delta
    products added in place by the kernel.  Checked against dequantise-then-matmul in fp32
    (rel-L2 <= 1e-2, the tolerance of the layer outputs) and against the fused kernel on the
    same inputs (the two differ by one fp16 rounding of the base product)."""
    from deltazip_b200 import ops, synth
    dev = torch.device("cuda")
    n, k, slots, m = 1024, 1536, 5, 1500
    g = torch.Generator(device=dev).manual_seed(7)
    w = (torch.randn((n, k), generator=g, device=dev) * 0.02).half()
    x = torch.randn((m, k), generator=g, device=dev).half()
    qw, meta, sc = synth.random_delta_slots(slots, n, k, bits, seed=3, device=dev, std=1e-2)
    idx = torch.sort(torch.randint(-1, slots, (m,), generator=g, device=dev))[0]
    seg = ops.Segments(m, slots, dev).build(idx)
    assert m > ops.FUSED_MAX_TOKENS
    got = ops.sbmm(x, qw, sc, meta, seg, w)
    want = x.float() @ w.float().t()
    for s in range(slots):
        rows = (idx == s).nonzero().flatten()
        want[rows] += x[rows].float() @ ops.unpack(qw[s], meta[s], sc[s], n, k, bits).float().t()
    rel = ((got.float() - want).norm() / want.norm()).item()
    assert rel <= 1e-2, rel
    keep = ops.FUSED_MAX_TOKENS
    try:
        ops.FUSED_MAX_TOKENS = 1 << 30
        fused = ops.sbmm(x, qw, sc, meta, seg, w)
    finally:
        ops.FUSED_MAX_TOKENS = keep
    rel2 = ((got.float() - fused.float()).norm() / fused.float().norm()).item()
    assert rel2 <= 2e-3, rel2
    # into a column slice of a wider tensor, and the base product alone
    wide = torch.zeros((m, n + 256), device=dev, dtype=torch.float16)
    ops.sbmm(x, qw, sc, meta, seg, w, out=wide[:, 128:128 + n])
    assert torch.equal(wide[:, 128:128 + n], got) and not wide[:, :128].any() and not wide[:, 128 + n:].any()
    base = ops.base_gemm(x, w)
    assert ((base.float() - x.float() @ w.float().t()).norm() / want.norm()).item() <= 2e-3
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [2, 4])
def test_prefill_runs_known_on_the_host_take_the_dequantise_once_path(bits):
    """A sorted prefill-sized batch whose runs the caller knows (Segments.host_runs, as the slot
    manager provides) multiplies each long run by the slot's dequantised delta through the
    library GEMM; the result must agree with the kernel path and with the fp32 reference."""
    from deltazip_b200 import ops, synth
    dev = torch.device("cuda")
    n, k, slots = 1024, 1024, 3
    lens = [300, 600, 256, 400]                      # base rows, slot 0, slot 1, slot 2
    idx = torch.cat([torch.full((c,), s - 1, dtype=torch.int64) for s, c in enumerate(lens)]).to(dev)
    m = idx.numel()
    g = torch.Generator(device=dev).manual_seed(11)
    w = (torch.randn((n, k), generator=g, device=dev) * 0.02).half()
    x = torch.randn((m, k), generator=g, device=dev).half()
    qw, meta, sc = synth.random_delta_slots(slots, n, k, bits, seed=5, device=dev, std=1e-2)
    seg = ops.Segments(m, slots, dev).build(idx, sorted_hint=True)
    kernel_path = ops.sbmm(x, qw, sc, meta, seg, w)
    edges = [0]
    for c in lens:
        edges.append(edges[-1] + c)
    seg.host_runs = [(s - 1, edges[s], edges[s + 1]) for s in range(len(lens))]
    dense_path = ops.sbmm(x, qw, sc, meta, seg, w)
    want = x.float() @ w.float().t()
    for s in range(slots):
        rows = (idx == s).nonzero().flatten()
        want[rows] += x[rows].float() @ ops.unpack(qw[s], meta[s], sc[s], n, k, bits).float().t()
    assert ((dense_path.float() - want).norm() / want.norm()).item() <= 2e-3
    assert ((dense_path.float() - kernel_path.float()).norm() / want.norm()).item() <= 2e-3
    # a short run sends the whole call back to the kernel
    seg.host_runs = [(-1, 0, 300), (0, 300, 900), (1, 900, 1000), (1, 1000, 1156), (2, 1156, m)]
    again = ops.sbmm(x, qw, sc, meta, seg, w)
    assert torch.equal(again, kernel_path)
    # the slot manager's mapping yields the runs for such a batch
    from deltazip_b200.models import DeltaMapping, _convert_mapping
    ids = [0] * 300 + [7] * 600 + [9] * 700
    _, (is_sorted, runs) = _convert_mapping(DeltaMapping(ids, [0, 7, 9]), [7, 9, None], 4, 32000, 0, device=dev)
    assert is_sorted and runs == [(-1, 0, 300), (0, 300, 900), (1, 900, 1600)]
