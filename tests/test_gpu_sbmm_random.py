"""Randomised parity of the SBMM against a dense evaluation on the same device.

Shapes, token counts, slot counts, bit widths and token orders are drawn from a seeded generator
so that odd combinations are exercised too: a 64-wide k tail, more tokens than one token block,
tiles split over many CTAs, slots without tokens, all-base batches.  The reference is the
library's own `unpack` (bit-exact against the reference's QuantLinear.unpack in
tests/test_gpu_format.py) followed by fp32 matmuls, i.e. the dequantise-then-matmul path.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dense_reference(x, w, dense, idx):
    y = x.float() @ w.float().t()
    for s in range(dense.shape[0]):
        rows = (idx == s).nonzero().flatten()
        if rows.numel():
            y[rows] += x[rows].float() @ dense[s].float().t()
    return y


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_shapes_against_dense(seed):
    from deltazip_b200 import ops, synth
    rng = np.random.default_rng(1000 + seed)
    bits = int(rng.choice([2, 4]))
    n = 128 * int(rng.integers(1, 40))
    k = 64 * int(rng.integers(1, 70))
    slots = int(rng.integers(1, 12))
    m = int(rng.choice([1, 3, 16, 17, 64, 100, 128, 129, 200, 300]))
    dtype = torch.float16 if seed % 3 else torch.bfloat16
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    w = (torch.randn((n, k), generator=g, device=dev) * 0.02).to(dtype)
    x = torch.randn((m, k), generator=g, device=dev).to(dtype)
    qw, meta, sc = synth.random_delta_slots(slots, n, k, bits, seed=seed, device=dev, std=1e-2)
    idx = torch.from_numpy(rng.integers(-1, slots, size=m)).to(dev)
    if seed % 4 == 0:
        idx, _ = torch.sort(idx)
    if seed == 5:
        idx[:] = -1
    dense = torch.stack([ops.unpack(qw[s], meta[s], sc[s], n, k, bits) for s in range(slots)])
    want = _dense_reference(x, w, dense, idx)
    got = ops.apply_delta(x, qw, sc, meta, idx, w).float()
    torch.cuda.synchronize()
    assert ops.read_status(x.device) == 0
    rel = ((got - want).norm() / want.norm().clamp_min(1e-6)).item()
    tol = 1e-2 if dtype == torch.float16 else 2e-2     # bf16 keeps 8 bits of mantissa
    assert rel <= tol, (seed, bits, n, k, slots, m, dtype, rel)
    # delta-only form on the same inputs
    only = ops.sbmm(x, qw, sc, meta, ops.Segments(m, slots, dev).build(idx), None).float()
    base = ops.base_gemm(x, w).float()
    torch.cuda.synchronize()
    rel2 = ((only + base - want).norm() / want.norm().clamp_min(1e-6)).item()
    assert rel2 <= 2 * tol, (seed, rel2)
