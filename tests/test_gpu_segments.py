"""The device-built segment table against a numpy restatement of its rules."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def expected_windows(idx, num_slots, token_block=128, max_cols=32):
    idx = np.where((idx >= num_slots) | (idx < -1), -1, idx)
    order = np.sort(idx, kind="stable")
    wins = []
    for s in range(num_slots):
        pos = np.nonzero(order == s)[0]
        if len(pos) == 0:
            continue
        s0, e0 = int(pos[0]), int(pos[-1]) + 1
        while s0 < e0:
            tb = s0 // token_block
            pe = min(e0, (tb + 1) * token_block)
            c0, c1 = s0 & ~15, (pe + 15) & ~15
            while c0 < c1:
                nc = min(max_cols, c1 - c0)
                wins.append((s, c0, nc, max(s0, c0), min(pe, c0 + nc)))
                c0 += nc
            s0 = pe
    return order, wins


@pytest.mark.parametrize("m,slots,sort,seed", [(64, 8, True, 0), (300, 5, True, 1), (1000, 64, False, 2),
                                               (1, 1, True, 3), (257, 3, False, 4), (4096, 2, True, 5)])
def test_segment_table(m, slots, sort, seed):
    from deltazip_b200 import ops
    from deltazip_b200._lib import lib
    rng = np.random.default_rng(seed)
    idx = rng.integers(-1, slots, size=m).astype(np.int64)
    if sort:
        idx = np.sort(idx)
    seg = ops.Segments(m, slots, "cuda").build(torch.from_numpy(idx).cuda())
    hdr = seg.header()
    order, wins = expected_windows(idx, slots)
    is_sorted = bool((np.diff(idx) >= 0).all())
    assert hdr[0] == m and hdr[1] == slots and hdr[2] == (m + 127) // 128
    assert hdr[3] == int(is_sorted) and hdr[4] == 0
    assert hdr[5] == len(wins) and hdr[6] == len(set(idx[idx >= 0].tolist()))
    raw = seg.buf.cpu().numpy()
    mr = (max(m, 1) + 63) // 64 * 64
    perm = raw[64:64 + 4 * mr].view(np.int32)[:m]
    slot_of = raw[64 + 4 * mr:64 + 8 * mr].view(np.int32)[:m]
    assert sorted(perm.tolist()) == list(range(m))
    np.testing.assert_array_equal(slot_of, order)
    np.testing.assert_array_equal(idx[perm], order)
    if is_sorted:
        np.testing.assert_array_equal(perm, np.arange(m))
    nb = (m + 127) // 128
    off = 64 + 8 * mr
    bb = raw[off:off + 4 * ((nb + 2 + 15) // 16 * 16)].view(np.int32)
    off += 4 * ((nb + 2 + 15) // 16 * 16)
    w = raw[off:off + 32 * len(wins)].view(np.int32).reshape(-1, 8)[:, :5]
    assert [tuple(r) for r in w.tolist()] == wins
    for tb in range(nb + 1):
        assert bb[tb] == sum(1 for x in wins if x[1] < tb * 128)
    assert lib().dz_segments_bytes(m, slots) == seg.buf.numel()
