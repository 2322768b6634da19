"""GPU parity of the format kernels: converter bytes equal the numpy restatement
of the slot layout, and unpack is bit-exact against the reference's unpack
(golden vectors) and the oracle (seeded synthetic layers)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import deltazip_oracle as O
from oracle import slot_layout as S

pytestmark = pytest.mark.gpu

CASES = [c for c in sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "b[0-9]*.npz")))
         if "b8" not in c]


def _to_dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(c)[:-4] for c in CASES])
def test_convert_unpack_golden(path):
    from deltazip_b200 import ops
    c = dict(np.load(path))
    bits = int(c["bits"])
    n, k = c["dense"].shape
    sq, sm, ss = ops.convert_from_gptq(_to_dev(c["qweight"]), _to_dev(c["qzeros"]),
                                       _to_dev(c["scales"]), bits)
    eq, em, es = S.to_slot(c["qweight"], c["qzeros"], c["scales"], bits)
    np.testing.assert_array_equal(sq.cpu().numpy(), eq)
    np.testing.assert_array_equal(sm.cpu().numpy(), em)
    np.testing.assert_array_equal(ss.cpu().numpy().view(np.uint16), es.view(np.uint16))
    d = ops.unpack(sq, sm, ss, n, k, bits).cpu().numpy()
    np.testing.assert_array_equal(d.view(np.uint16), c["dense"].view(np.uint16))


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("n,k", [(128, 64), (384, 448), (1024, 1024)])
def test_convert_unpack_synthetic(bits, n, k):
    from deltazip_b200 import ops
    _, deltas = O.make_layer(n, k, 1, bits, seed=n + k + bits)
    qw, qz, sc, _ = deltas[0]
    sq, sm, ss = ops.convert_from_gptq(_to_dev(qw), _to_dev(qz), _to_dev(sc), bits)
    d = ops.unpack(sq, sm, ss, n, k, bits).cpu().numpy()
    np.testing.assert_array_equal(d.view(np.uint16), O.unpack(qw, qz, sc, bits).view(np.uint16))


def test_converter_flags_dense_input():
    """A delta that is not 2:4 sparse is reported, not silently truncated."""
    from deltazip_b200 import ops, DeltaZipError
    from deltazip_b200 import _lib
    rng = np.random.default_rng(0)
    d = rng.standard_normal((128, 64), dtype=np.float32) * 1e-3
    scale, zero, maxq = O.find_params_sym(d, 4)
    wq = O.quantize_values(d, scale, zero, maxq)          # no pruning
    qw, qz, sc = O.pack(wq, scale, zero, 4)
    with pytest.raises(DeltaZipError) as e:
        ops.convert_from_gptq(_to_dev(qw), _to_dev(qz), _to_dev(sc), 4)
    assert e.value.status == _lib.DZ_ERR_NOT_2_4


def test_converter_flags_asymmetric_zero_point():
    from deltazip_b200 import ops, DeltaZipError
    from deltazip_b200 import _lib
    _, deltas = O.make_layer(128, 64, 1, 4, seed=1)
    qw, qz, sc, _ = deltas[0]
    qz = qz.copy()
    qz[0, 0] ^= 0x3
    with pytest.raises(DeltaZipError) as e:
        ops.convert_from_gptq(_to_dev(qw), _to_dev(qz), _to_dev(sc), 4)
    assert e.value.status == _lib.DZ_ERR_NOT_SYMMETRIC


@pytest.mark.parametrize("bits", [2, 4])
def test_gpu_compressor_matches_oracle(bits):
    """The torch-op compressor used to build benchmark-size inputs produces the
    same GPTQ tensors as the oracle's restatement of the reference pipeline."""
    from deltazip_b200 import synth
    rng = np.random.default_rng(5)
    d = rng.standard_normal((256, 512), dtype=np.float32) * np.float32(1e-3)
    d[3] = 0
    wq, scale, zero = O.compress_delta(d, bits)
    qw, qz, sc = O.pack(wq, scale, zero, bits)
    gqw, gqz, gsc = synth.compress_delta_gptq(_to_dev(d), bits)
    np.testing.assert_array_equal(gqw.cpu().numpy(), qw)
    np.testing.assert_array_equal(gqz.cpu().numpy(), qz)
    np.testing.assert_array_equal(gsc.cpu().numpy().view(np.uint16), sc.view(np.uint16))
