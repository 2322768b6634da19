"""The numpy restatement of the slot layout round-trips and reproduces the
reference's unpack on the golden GPTQ tensors."""
import glob
import os

import numpy as np
import pytest

from oracle import deltazip_oracle as O
from oracle import slot_layout as S

CASES = [c for c in sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "b[0-9]*.npz")))
         if "b8" not in c]


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(c)[:-4] for c in CASES])
def test_slot_roundtrip_golden(path):
    c = dict(np.load(path))
    bits = int(c["bits"])
    n, k = c["dense"].shape
    if n % 128 or k % 64:
        pytest.skip("shape outside the slot layout")
    sq, sm, ss = S.to_slot(c["qweight"], c["qzeros"], c["scales"], bits)
    assert sq.shape == (k * bits // 128, 2 * n) and sm.shape == (n, k // 16)
    d = S.from_slot(sq, sm, ss, n, k, bits)
    np.testing.assert_array_equal(d.view(np.uint16), c["dense"].view(np.uint16))


def test_kept_pair_rule():
    nz = np.array([[0, 0, 0, 0], [1, 0, 0, 0], [0, 0, 0, 1], [0, 1, 0, 0], [0, 1, 1, 0],
                   [1, 0, 0, 1], [0, 0, 1, 1]], dtype=bool)
    i0, i1 = S.kept_pairs(nz)
    assert list(zip(i0, i1)) == [(0, 1), (0, 1), (0, 3), (0, 1), (1, 2), (0, 3), (2, 3)]
    with pytest.raises(ValueError):
        S.kept_pairs(np.array([[1, 1, 1, 0]], dtype=bool))
