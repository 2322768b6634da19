"""CPU restatement of the library's slot layout (TEST INFRASTRUCTURE ONLY).

The slot layout is this repository's own design (the reference fixes only the
names, dtypes and outer shapes of the slot tensors,
serving/vllm/delta/layers_marlin.py:311-333); this numpy version states it a
second time, independently of the CUDA index functions in
deltazip_b200/csrc/dz_common.cuh, so that the converter's bytes can be checked.
"""
from __future__ import annotations

import numpy as np

from . import deltazip_oracle as O

TILE_N = 128
BLOCK_K = 64


def kept_pairs(nz: np.ndarray):
    """nz: bool [..., 4] (code != zero-point).  Returns (i0, i1) int arrays [...],
    i0 < i1: the non-zero positions ascending, filled up with the lowest-index
    remaining positions and re-sorted when fewer than two are non-zero."""
    cnt = nz.sum(axis=-1)
    if (cnt > 2).any():
        raise ValueError("not 2:4 sparse")
    pos = np.arange(4)
    # rank positions: non-zero first (ascending), then zero positions ascending
    key = np.where(nz, pos, pos + 4)
    order = np.argsort(key, axis=-1, kind="stable")[..., :2]
    order = np.sort(order, axis=-1)
    return order[..., 0], order[..., 1]


def to_slot(qweight: np.ndarray, qzeros: np.ndarray, scales: np.ndarray, bits: int):
    """GPTQ-layout tensors -> (slot_qweight int32 [K*bits/128, 2N], slot_meta int16 [N, K/16],
    slot_scales fp16 [1, N])."""
    q, z = O.unpack_codes(qweight, qzeros, bits)      # q [K, N], z [N]
    k, n = q.shape
    assert n % TILE_N == 0 and k % BLOCK_K == 0
    if not (z == (1 << (bits - 1))).all():
        raise ValueError("zero-point is not symmetric")
    qt = q.T.reshape(n, k // 4, 4)                     # [N, G, 4]
    nz = qt != z[:, None, None]
    i0, i1 = kept_pairs(nz)                            # [N, G]
    c0 = np.take_along_axis(qt, i0[..., None], axis=2)[..., 0].astype(np.uint32)
    c1 = np.take_along_axis(qt, i1[..., None], axis=2)[..., 0].astype(np.uint32)
    num_kb = k // BLOCK_K
    codes = np.stack([c0, c1], axis=-1).reshape(n, num_kb, 32)        # kept value e = 2g + which
    per = 32 // bits
    words = np.zeros((n, num_kb, bits), dtype=np.uint32)              # `bits` words per row-block
    for e in range(32):
        el = e % per
        shift = (el & 1) * 16 + bits * (el >> 1)
        words[:, :, e // per] |= codes[:, :, e] << np.uint32(shift)
    # [tile][kb][row][words]
    sq = words.reshape(n // TILE_N, TILE_N, num_kb, bits).transpose(0, 2, 1, 3)
    sq = np.ascontiguousarray(sq).reshape(-1).view(np.int32).reshape(k * bits // 128, 2 * n)

    nib = (i0 | (i1 << 2)).astype(np.uint32).reshape(n, num_kb, 2, 2, 4)   # [n, kb, c, kh, gg]
    h16 = np.zeros((n, num_kb, 2, 2), dtype=np.uint32)
    for gg in range(4):
        h16 |= nib[..., gg] << np.uint32(4 * gg)
    meta = np.zeros((n // TILE_N, num_kb, TILE_N, 2, 2), dtype=np.uint16)  # [t, kb, lane, c, half]
    r = np.arange(TILE_N)
    half = (r >> 3) & 1
    h16 = h16.reshape(n // TILE_N, TILE_N, num_kb, 2, 2)                   # [t, r, kb, c, kh]
    for kh in range(2):
        lane = (r & 7) + 8 * kh + 16 * (r >> 4)
        for c in range(2):
            meta[:, :, lane, c, half] = h16[:, :, :, c, kh].transpose(0, 2, 1).astype(np.uint16)
    sm = meta.reshape(-1).view(np.int16).reshape(n, k // 16)
    return sq, sm, np.asarray(scales, np.float16).reshape(1, n).copy()


def from_slot(sq: np.ndarray, sm: np.ndarray, ss: np.ndarray, n: int, k: int, bits: int) -> np.ndarray:
    """Slot tensors -> dense fp16 delta [N, K]."""
    num_kb = k // BLOCK_K
    per = 32 // bits
    maxq = (1 << bits) - 1
    words = np.ascontiguousarray(sq).reshape(-1).view(np.uint32)
    words = words.reshape(n // TILE_N, num_kb, TILE_N, bits).transpose(0, 2, 1, 3).reshape(n, num_kb, bits)
    codes = np.zeros((n, num_kb, 32), dtype=np.int32)
    for e in range(32):
        el = e % per
        shift = (el & 1) * 16 + bits * (el >> 1)
        codes[:, :, e] = (words[:, :, e // per] >> np.uint32(shift)) & maxq
    meta = np.ascontiguousarray(sm).reshape(-1).view(np.uint16).reshape(n // TILE_N, num_kb, TILE_N, 2, 2)
    r = np.arange(TILE_N)
    half = (r >> 3) & 1
    h16 = np.zeros((n // TILE_N, TILE_N, num_kb, 2, 2), dtype=np.uint32)
    for kh in range(2):
        lane = (r & 7) + 8 * kh + 16 * (r >> 4)
        for c in range(2):
            h16[:, :, :, c, kh] = meta[:, :, lane, c, half].transpose(0, 2, 1)
    h16 = h16.reshape(n, num_kb, 2, 2)
    s = np.asarray(ss, np.float16).reshape(-1).astype(np.float32)
    z = 1 << (bits - 1)
    dense = np.zeros((n, num_kb, 16, 4), dtype=np.float16)
    rows = np.arange(n)[:, None]
    kbs = np.arange(num_kb)[None, :]
    for c in range(2):
        for kh in range(2):
            for gg in range(4):
                g = c * 8 + kh * 4 + gg
                nibv = (h16[:, :, c, kh] >> np.uint32(4 * gg)) & 0xF
                i0 = (nibv & 3).astype(np.int64)
                i1 = ((nibv >> 2) & 3).astype(np.int64)
                v0 = (s[:, None] * (codes[:, :, 2 * g] - z).astype(np.float32)).astype(np.float16)
                v1 = (s[:, None] * (codes[:, :, 2 * g + 1] - z).astype(np.float32)).astype(np.float16)
                dense[rows, kbs, g, i0] = v0
                same = i0 == i1
                dense[rows, kbs, g, i1] = np.where(same, dense[rows, kbs, g, i1], v1)
    return dense.reshape(n, k)
