"""Full-output parity of the SBMM on the shapes the benchmark runs.

Every launch shape of the benchmark configurations is compared, all outputs, with the
dequantise-then-matmul path evaluated on the same device: `ops.unpack` (bit-exact against the
reference's QuantLinear.unpack, tests/test_gpu_format.py) gives the dense fp16 delta, and
y = x W^T + x delta^T is formed in float32.  Covered on purpose:
  * 22016 x 4096 -- more 128-row tiles (172) than CTAs, so a CTA finishes one tile, runs whole
    tiles and starts another;
  * 4096 x 11008 -- 86 k-units per tile, tiles split over five to six CTAs;
  * the single-layer configuration exactly (4096 x 4096, one 2-bit delta, 16 tokens, seed 0)
    against the CPU oracle;
  * many-delta batches: 32 slots / 128 tokens and 64 slots / 256 tokens (two token blocks), 2-bit.
Tolerance: rel-L2 <= 1e-2 over the batch (the stated bar for fp16 layer outputs), 2e-2 for any
single token, and 2e-3 against the float32 value (the fused kernel rounds once).
"""
import numpy as np
import pytest
import torch

from oracle import deltazip_oracle as O
from tests.gpu_util import DeviceLayer, dev

pytestmark = pytest.mark.gpu
TOL = 1e-2


def dense_reference(x, w, qw, meta, sc, idx, bits):
    """float32 y = x W^T + x dequant(delta_slot)^T on the device, one slot at a time."""
    from deltazip_b200 import ops
    n, k = w.shape
    y = x.float() @ w.float().t()
    for s in torch.unique(idx).tolist():
        if s < 0:
            continue
        rows = (idx == s).nonzero().flatten()
        dense = ops.unpack(qw[s], meta[s], sc[s], n, k, bits)
        y[rows] += x[rows].float() @ dense.float().t()
        del dense
    return y


def compare(got, want, idx):
    got = got.float()
    assert torch.isfinite(got).all()
    rel = ((got - want).norm() / want.norm()).item()
    assert rel <= 2e-3, f"rel-L2 {rel} against the float32 value"
    per_row = (got - want).norm(dim=1) / want.norm(dim=1).clamp_min(1e-6)
    worst = int(per_row.argmax())
    assert per_row[worst].item() <= 2 * TOL, f"token {worst} (slot {int(idx[worst])}): {per_row[worst].item()}"
    return rel


BENCH_SHAPES = [("qkv_proj", 12288, 4096), ("o_proj", 4096, 4096),
                ("gate_up_proj", 22016, 4096), ("down_proj", 4096, 11008)]


@pytest.mark.parametrize("name,n,k", BENCH_SHAPES)
def test_benchmark_launch_shapes_all_outputs(name, n, k):
    """The four launches of the SBMM benchmark: 8 deltas, 4-bit, 64 sorted tokens."""
    from deltazip_b200 import ops, synth
    d = torch.device("cuda")
    g = torch.Generator(device=d).manual_seed(n + k)
    w = (torch.randn((n, k), generator=g, device=d) * 0.02).half()
    x = torch.randn((64, k), generator=g, device=d).half()
    qw, meta, sc = synth.random_delta_slots(8, n, k, 4, seed=n ^ k, device=d)
    idx = torch.sort(torch.randint(0, 8, (64,), generator=g, device=d))[0]
    seg = ops.Segments(64, 8, d).build(idx, sorted_hint=True)
    y = ops.sbmm(x, qw, sc, meta, seg, w, bits=4)
    torch.cuda.synchronize()
    assert ops.read_status(d) == 0
    compare(y, dense_reference(x, w, qw, meta, sc, idx, 4), idx)
    # the same launch again is bit-identical (fixed summation order over the split tiles)
    y2 = ops.sbmm(x, qw, sc, meta, seg, w, bits=4)
    assert torch.equal(y, y2)
    # and the drop-in op (no promise about the order, no host synchronisation) agrees bit for bit
    y3 = ops.apply_delta(x, qw, sc, meta, idx, w)
    assert torch.equal(y, y3)


def test_single_layer_configuration_against_the_oracle():
    """4096 x 4096 base ~ N(0, 0.02), one delta ~ N(0, 1e-3) 2:4-pruned, 2-bit symmetric per-row
    scale, x [16, 4096] ~ N(0, 1), seed 0: the CPU-runnable configuration, end to end through the
    oracle's quantiser, packer and dequantise-then-matmul."""
    layer = DeviceLayer(4096, 4096, 1, 2, seed=0)
    x, _ = O.make_tokens(16, 4096, 1, seed=0)
    idx = np.zeros(16, dtype=np.int64)
    from deltazip_b200 import ops
    seg = ops.Segments(16, 1, "cuda").build(dev(idx), sorted_hint=True)
    y = ops.sbmm(dev(x), layer.qweight, layer.scales, layer.meta, seg, layer.w).cpu().numpy()
    ref = layer.oracle(x, idx)                       # fp16(base) + fp16(delta), as the reference adds
    assert O.rel_l2(y, ref) <= TOL
    assert O.rel_l2(y, layer.oracle_fp32(x, idx)) <= 2e-3
    for i in range(16):
        assert O.rel_l2(y[i], ref[i]) <= 2 * TOL
    # the delta part alone, so that a wrong delta cannot hide behind the (20x larger) base output
    only = ops.sbmm(dev(x), layer.qweight, layer.scales, layer.meta, seg, None).float().cpu().numpy()
    want = x.astype(np.float32) @ layer.dense()[0].astype(np.float32).T
    assert O.rel_l2(only, want) <= 2e-3


@pytest.mark.parametrize("n,k,slots,m,zipf", [(12288, 4096, 32, 128, False),
                                             (15360, 5120, 64, 256, True),
                                             (5120, 13824, 64, 256, True)])
def test_many_delta_batches_two_bit(n, k, slots, m, zipf):
    """32 resident 2-bit deltas / 128 sequences (7B qkv) and 64 deltas / 256 sequences with a
    Zipf(1.5) request-to-delta map (13B qkv and down_proj): token blocks wider than 64 columns,
    two token blocks, slots with a single token and slots with none."""
    from deltazip_b200 import ops, synth
    d = torch.device("cuda")
    g = torch.Generator(device=d).manual_seed(m + slots)
    w = (torch.randn((n, k), generator=g, device=d) * 0.02).half()
    x = torch.randn((m, k), generator=g, device=d).half()
    qw, meta, sc = synth.random_delta_slots(slots, n, k, 2, seed=slots, device=d)
    if zipf:
        p = 1.0 / torch.arange(1, slots + 1, dtype=torch.float64) ** 1.5
        idx = torch.multinomial(p / p.sum(), m, replacement=True,
                                generator=torch.Generator().manual_seed(5)).to(d)
    else:
        idx = torch.randint(0, slots, (m,), generator=g, device=d)
    idx = torch.sort(idx)[0]
    seg = ops.Segments(m, slots, d).build(idx, sorted_hint=True)
    y = ops.sbmm(x, qw, sc, meta, seg, w, bits=2)
    torch.cuda.synchronize()
    assert ops.read_status(d) == 0
    compare(y, dense_reference(x, w, qw, meta, sc, idx, 2), idx)
    # delta-only output of the same batch, compared on its own scale
    only = ops.sbmm(x, qw, sc, meta, seg, None, bits=2).float()
    want = dense_reference(x, torch.zeros_like(w), qw, meta, sc, idx, 2)
    assert ((only - want).norm() / want.norm()).item() <= 2e-3


def test_in_place_slices_of_a_merged_output_full_width():
    """add_delta_slice at benchmark width: q, k and v stacks (4096 rows each) added in place into
    the column slices of one [64, 12288] base output through the kernel's row stride."""
    from deltazip_b200 import ops, synth
    d = torch.device("cuda")
    g = torch.Generator(device=d).manual_seed(3)
    k, widths = 4096, (4096, 4096, 4096)
    x = torch.randn((64, k), generator=g, device=d).half()
    idx = torch.sort(torch.randint(-1, 4, (64,), generator=g, device=d))[0]
    out = (torch.randn((64, sum(widths)), generator=g, device=d) * 0.5).half()
    want = out.float().clone()
    stacks, off = [], 0
    for i, wd in enumerate(widths):
        qw, meta, sc = synth.random_delta_slots(4, wd, k, 4, seed=70 + i, device=d, std=1e-2)
        stacks.append((qw, meta, sc))
        want[:, off:off + wd] += dense_reference(x, torch.zeros((wd, k), device=d, dtype=torch.half),
                                                 qw, meta, sc, idx, 4)
        off += wd
    ops.apply_delta_packed_nslice(x, [s[0] for s in stacks], None, [s[2] for s in stacks], None,
                                  idx, out, widths, meta_stacked=[s[1] for s in stacks])
    torch.cuda.synchronize()
    assert ops.read_status(d) == 0
    assert ((out.float() - want).norm() / want.norm()).item() <= 2e-3
