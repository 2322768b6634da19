"""CPU oracle for the DeltaZip selective-batched-matmul (SBMM) path.

TEST INFRASTRUCTURE ONLY.  This module is a numpy restatement of the reference's
algorithm and is the checker the CUDA path is compared against.  Nothing in the
shipped package may import it; only tests, the smoke check and the CPU-baseline
leg of the benchmark do.

Parity pin: every function below that restates reference code is checked against
outputs of that reference code (loaded by file path, run on CPU) stored under
tests/golden/ -- see tests/golden/make_golden.py and tests/test_oracle_golden.py.
The production SBMM kernel of the reference lives in the un-vendored, un-pinned
third-party package ``triteia`` (eth-easl/triteia at HEAD; call site
serving/vllm/delta/deltazip_marlin.py:18) whose source is absent, and the
reference has no tests for this path, so parity AT THE SBMM OP BOUNDARY is
unpinned; what is pinned is the in-tree PyTorch dequantise-then-matmul path the
op must agree with.

Reference citations (paths relative to the reference checkout):
  find_params_sym   deltazip/core/quant.py:48-86
  quantize_codes    deltazip/core/quant.py:9-18
  mask_2_4          deltazip/core/sparsegpt.py:123-125 (with H = I)
  pack              deltazip/nn_modules/qlinear.py:83-183
  unpack            deltazip/nn_modules/qlinear.py:185-264
  delta_forward     deltazip/nn_modules/qlinear.py:266-341
  base_linear       serving/vllm/model_executor/layers/linear.py:85-96
  apply_delta       serving/vllm/delta/deltazip.py:24-30,
                    serving/vllm/delta/deltazip_marlin.py:10-19,44-53
  row_parallel      serving/vllm/delta/layers_marlin.py:573-597
"""
from __future__ import annotations

import numpy as np

# --------------------------------------------------------------------------
# Quantisation grid, 2:4 mask (input generators for the path)
# --------------------------------------------------------------------------


def find_params_sym(w: np.ndarray, bits: int):
    """Per-output-row symmetric grid.  w: [N, K] float32.

    Returns (scale[N] float32, zero[N] float32, maxq).  Follows
    Quantizer.find_params with perchannel=True, sym=True, weight=True:
    xmin/xmax are clamped through 0, the larger magnitude is mirrored when the
    row has a negative entry, an all-zero row gets the range [-1, 1],
    scale = (xmax - xmin) / maxq and zero = (maxq + 1) / 2.
    """
    w = np.asarray(w, dtype=np.float32)
    maxq = (1 << bits) - 1
    xmin = np.minimum(w.min(axis=1), np.float32(0))
    xmax = np.maximum(w.max(axis=1), np.float32(0))
    xmax = np.maximum(np.abs(xmin), xmax)
    neg = xmin < 0
    xmin = np.where(neg, -xmax, xmin)
    dead = (xmin == 0) & (xmax == 0)
    xmin = np.where(dead, np.float32(-1), xmin)
    xmax = np.where(dead, np.float32(1), xmax)
    scale = ((xmax - xmin) / np.float32(maxq)).astype(np.float32)
    zero = np.full_like(scale, (maxq + 1) / 2, dtype=np.float32)
    return scale, zero, maxq


def quantize_codes(w: np.ndarray, scale: np.ndarray, zero: np.ndarray, maxq: int):
    """Integer codes q = clamp(round(w / scale) + zero, 0, maxq), round-half-even.

    w: [N, K] float32, scale/zero: [N].  Returns int32 [N, K].
    """
    q = np.rint(np.asarray(w, np.float32) / scale[:, None]) + zero[:, None]
    return np.clip(q, 0, maxq).astype(np.int32)


def quantize_values(w, scale, zero, maxq):
    """The de-quantised float the reference's ``quantize`` returns: scale*(q-zero)."""
    q = quantize_codes(w, scale, zero, maxq).astype(np.float32)
    return (scale[:, None] * (q - zero[:, None])).astype(np.float32)


def mask_2_4(w: np.ndarray) -> np.ndarray:
    """Boolean keep-mask [N, K]: in every 4 consecutive K keep the 2 largest |w|.

    The reference prunes the 2 entries with the smallest w^2 / diag(Hinv)^2 per
    group; with no calibration data H = I this is "drop the two smallest
    magnitudes".  Ties are broken towards keeping the lower index (stable sort);
    the generators in this repo draw float32 deltas so ties do not occur.
    """
    w = np.asarray(w, np.float32)
    n, k = w.shape
    g = (w.reshape(n, k // 4, 4).astype(np.float64)) ** 2
    order = np.argsort(-g, axis=2, kind="stable")  # descending magnitude
    keep = np.zeros_like(g, dtype=bool)
    np.put_along_axis(keep, order[:, :, :2], True, axis=2)
    return keep.reshape(n, k)


def compress_delta(delta: np.ndarray, bits: int):
    """2:4 prune then symmetric per-row quantise (the compression the configs name).

    Mirrors the order inside SparseGPT.fasterprune with H = I and no error
    feedback: the quantiser grid is found on the *dense* delta
    (deltazip/core/sparsegpt.py:62-64), pruned entries are set to 0 and then
    every entry goes through ``quantize`` (sparsegpt.py:127-136).

    Returns (wq float32 [N,K] de-quantised values, scale[N], zero[N]).
    """
    delta = np.asarray(delta, np.float32)
    scale, zero, maxq = find_params_sym(delta, bits)
    keep = mask_2_4(delta)
    pruned = np.where(keep, delta, np.float32(0))
    wq = quantize_values(pruned, scale, zero, maxq)
    return wq, scale, zero


# --------------------------------------------------------------------------
# GPTQ-style pack / unpack (the on-disk code layout and the bit-exactness target)
# --------------------------------------------------------------------------


def pack(wq: np.ndarray, scale: np.ndarray, zero: np.ndarray, bits: int):
    """QuantLinear.pack for bits in {2,4,8}, one quantisation group (g_idx == 0).

    wq: [N, K] float32 (values on the grid), scale/zero: [N] float32.
    Returns qweight int32 [K*bits/32, N], qzeros int32 [1, N*bits/32],
    scales float16 [1, N].

    intweight[k, n] = round((wq[n,k] + zero*scale) / fp16(scale)) computed the
    way torch does it there: float32 numerator divided by a float16 divisor
    promoted to float32, round-half-even, truncated to int32.
    """
    assert bits in (2, 4, 8)
    wq = np.asarray(wq, np.float32)
    n, k = wq.shape
    per = 32 // bits
    scale = np.asarray(scale, np.float32)
    zero = np.asarray(zero, np.float32)
    scale_zeros = (zero * scale).astype(np.float32)
    scales_h = scale.astype(np.float16)
    inty = np.rint((wq + scale_zeros[:, None]) / scales_h.astype(np.float32)[:, None])
    inty = inty.astype(np.int32).T.astype(np.uint32)  # [K, N]
    qweight = np.zeros((k // per, n), dtype=np.uint32)
    for j in range(per):
        qweight |= inty[j::per, :] << np.uint32(bits * j)
    z = (zero - 1).astype(np.uint32)  # stored zero-point is zero - 1
    qzeros = np.zeros((1, n // per), dtype=np.uint32)
    for j in range(per):
        qzeros[0] |= z[j::per] << np.uint32(bits * j)
    return qweight.view(np.int32), qzeros.view(np.int32), scales_h.reshape(1, n)


def unpack_codes(qweight: np.ndarray, qzeros: np.ndarray, bits: int):
    """Integer codes q[K, N] (0..maxq) and zero-points z[N] (stored value + 1)."""
    assert bits in (2, 4, 8)
    per = 32 // bits
    maxq = (1 << bits) - 1
    qw = np.ascontiguousarray(qweight).view(np.uint32)
    rows, n = qw.shape
    shifts = (np.arange(per, dtype=np.uint32) * np.uint32(bits))
    q = (qw[:, None, :] >> shifts[None, :, None]) & np.uint32(maxq)
    q = q.reshape(rows * per, n).astype(np.int32)
    qz = np.ascontiguousarray(qzeros).view(np.uint32)
    z = ((qz[:, :, None] >> shifts[None, None, :]) & np.uint32(maxq)).astype(np.int32) + 1
    return q, z.reshape(-1)


def unpack(qweight, qzeros, scales, bits: int) -> np.ndarray:
    """QuantLinear.unpack: dense delta [N, K] as float16 bit patterns.

    delta[n, k] = fp16( fp16(scale[n]) * (q[k, n] - z[n]) ): one float16 product
    of a float16 scale and a small exact integer, i.e. the correctly rounded
    float16 of the real product.  Computing it in float32 and rounding once to
    float16 gives the same bits (the float32 product of an 11-bit and a 4-bit
    significand is exact).
    """
    q, z = unpack_codes(qweight, qzeros, bits)
    s = np.asarray(scales, np.float16).reshape(-1).astype(np.float32)
    d = (s[None, :] * (q - z[None, :]).astype(np.float32)).astype(np.float16)  # [K, N]
    return np.ascontiguousarray(d.T)


# --------------------------------------------------------------------------
# Layer output
# --------------------------------------------------------------------------


def _mm_fp16(a16: np.ndarray, b16_t: np.ndarray) -> np.ndarray:
    """fp16 x fp16 matmul with float32 accumulation, result rounded to float16.

    a16: [M, K] float16, b16_t: [N, K] float16 -> [M, N] float16.
    """
    acc = a16.astype(np.float32) @ b16_t.astype(np.float32).T
    return acc.astype(np.float16)


def base_linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """F.linear(x, W) with no bias, fp16 in / fp16 out."""
    return _mm_fp16(np.asarray(x, np.float16), np.asarray(w, np.float16))


def delta_forward(x, qweight, qzeros, scales, bits) -> np.ndarray:
    """QuantLinear.forward: dequantise the whole delta, then matmul(x.half(), delta^T)."""
    return _mm_fp16(np.asarray(x, np.float16), unpack(qweight, qzeros, scales, bits))


def apply_delta(x, w_base, deltas, indices) -> np.ndarray:
    """y[i] = x[i] W^T + x[i] delta_{indices[i]}^T ; indices[i] == -1 -> base only.

    x: [M, K] fp16; w_base: [N, K] fp16; deltas: list of (qweight, qzeros,
    scales, bits) in GPTQ layout, one per slot (None = empty slot);
    indices: [M] ints.  The base output and the delta output are each rounded
    to fp16 and then added in fp16, as the reference's separate base GEMM +
    in-place delta add does (serving/vllm/delta/layers_unoptimized.py:275-288).
    """
    x = np.asarray(x, np.float16)
    y = base_linear(x, w_base)
    idx = np.asarray(indices).astype(np.int64)
    for d in np.unique(idx):
        if d < 0:
            continue
        rows = np.nonzero(idx == d)[0]
        qw, qz, sc, bits = deltas[int(d)]
        y[rows] = (y[rows] + delta_forward(x[rows], qw, qz, sc, bits)).astype(np.float16)
    return y


def apply_delta_dense(x, w_base, dense_deltas, indices) -> np.ndarray:
    """Same as apply_delta with pre-unpacked fp16 deltas [D][N, K] (float32 math,
    a single rounding at the end) -- the high-accuracy variant used as the
    "true value" when judging which of two fp16 results is closer."""
    x32 = np.asarray(x, np.float16).astype(np.float32)
    y = x32 @ np.asarray(w_base, np.float16).astype(np.float32).T
    idx = np.asarray(indices).astype(np.int64)
    for d in np.unique(idx):
        if d < 0:
            continue
        rows = np.nonzero(idx == d)[0]
        y[rows] += x32[rows] @ np.asarray(dense_deltas[int(d)], np.float16).astype(np.float32).T
    return y


def row_parallel_reduce(partials) -> np.ndarray:
    """Sum of per-rank fp16 partial outputs (tensor-parallel all-reduce), fp16 out.

    NCCL sums fp16 buffers in an implementation-defined order; the oracle sums
    in float32 and rounds once, and the test allows the fp16 tolerance."""
    acc = np.zeros(partials[0].shape, np.float32)
    for p in partials:
        acc += np.asarray(p, np.float16).astype(np.float32)
    return acc.astype(np.float16)


def rel_l2(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    den = float(np.sqrt((b * b).sum()))
    return float(np.sqrt(((a - b) ** 2).sum())) / (den if den > 0 else 1.0)


# --------------------------------------------------------------------------
# Seeded synthetic inputs with the shapes / distributions the benchmark configs name
# --------------------------------------------------------------------------


def make_layer(n: int, k: int, n_deltas: int, bits: int, seed: int = 0,
               w_std: float = 0.02, d_std: float = 1e-3):
    """Base W ~ N(0, w_std) fp16 [N,K]; n_deltas deltas ~ N(0, d_std) float32,
    2:4-pruned, symmetric `bits`-bit per-row, packed in GPTQ layout."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(w_std)).astype(np.float16)
    deltas = []
    for _ in range(n_deltas):
        d = rng.standard_normal((n, k), dtype=np.float32) * np.float32(d_std)
        wq, scale, zero = compress_delta(d, bits)
        qw, qz, sc = pack(wq, scale, zero, bits)
        deltas.append((qw, qz, sc, bits))
    return w, deltas


def make_tokens(m: int, k: int, n_slots: int, seed: int = 0, sort: bool = True,
                base_frac: float = 0.0):
    """x ~ N(0,1) fp16 [M,K]; slot ids uniform over n_slots (a fraction may be -1)."""
    rng = np.random.default_rng(seed + 1000003)
    x = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16)
    idx = rng.integers(0, max(n_slots, 1), size=m).astype(np.int64)
    if n_slots == 0:
        idx[:] = -1
    if base_frac > 0:
        idx[rng.random(m) < base_frac] = -1
    if sort:
        idx = np.sort(idx, kind="stable")
    return x, idx
