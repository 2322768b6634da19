"""Pins the CPU oracle to outputs of the reference's own code (tests/golden/*.npz,
produced by tests/golden/make_golden.py from deltazip/core/quant.py and
deltazip/nn_modules/qlinear.py run on CPU)."""
import glob
import os

import numpy as np
import pytest

from oracle import deltazip_oracle as O

# the pack / unpack / forward cases (the sparsegpt_* files hold the compressor's golden vectors and
# are read by tests/test_gpu_compress.py and test_sparsegpt_restatement below)
CASES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "b[0-9]*.npz")))


@pytest.fixture(params=CASES, ids=[os.path.basename(c)[:-4] for c in CASES])
def case(request):
    return dict(np.load(request.param))


def test_have_cases():
    assert len(CASES) >= 5


def test_grid_matches_reference(case):
    bits = int(case["bits"])
    scale, zero, maxq = O.find_params_sym(case["delta"], bits)
    np.testing.assert_array_equal(scale, case["scale"])
    np.testing.assert_array_equal(zero, case["zero"])
    assert maxq == 2 ** bits - 1


def test_mask_matches_reference(case):
    np.testing.assert_array_equal(O.mask_2_4(case["delta"]), case["keep"])


def test_quantised_values_match_reference(case):
    bits = int(case["bits"])
    wq, scale, zero = O.compress_delta(case["delta"], bits)
    np.testing.assert_array_equal(wq, case["wq"])


def test_pack_bit_exact(case):
    bits = int(case["bits"])
    qw, qz, sc = O.pack(case["wq"], case["scale"], case["zero"], bits)
    np.testing.assert_array_equal(qw, case["qweight"])
    np.testing.assert_array_equal(qz, case["qzeros"])
    np.testing.assert_array_equal(sc.view(np.uint16), case["scales"].view(np.uint16))


def test_unpack_bit_exact(case):
    bits = int(case["bits"])
    d = O.unpack(case["qweight"], case["qzeros"], case["scales"], bits)
    assert d.dtype == np.float16
    np.testing.assert_array_equal(d.view(np.uint16), case["dense"].view(np.uint16))


def test_forward_close_to_reference(case):
    bits = int(case["bits"])
    y = O.delta_forward(case["x"], case["qweight"], case["qzeros"], case["scales"], bits)
    # same fp16 operands; only the accumulation order inside the BLAS differs
    assert O.rel_l2(y, case["y_delta"]) <= 2e-3
    yb = O.base_linear(case["x"], case["w_base"])
    assert O.rel_l2(yb, case["y_base"]) <= 2e-3


def test_sparsity_is_2_4(case):
    bits = int(case["bits"])
    q, z = O.unpack_codes(case["qweight"], case["qzeros"], bits)
    nz = (q != z[None, :]).T  # [N, K]
    n, k = nz.shape
    assert nz.reshape(n, k // 4, 4).sum(axis=2).max() <= 2


def test_apply_delta_semantics():
    w, deltas = O.make_layer(128, 128, 3, 4, seed=5)
    x, idx = O.make_tokens(11, 128, 3, seed=5, base_frac=0.3)
    y = O.apply_delta(x, w, deltas, idx)
    for i in range(11):
        yi = O.base_linear(x[i:i + 1], w)
        if idx[i] >= 0:
            yi = (yi + O.delta_forward(x[i:i + 1], *deltas[idx[i]])).astype(np.float16)
        np.testing.assert_array_equal(y[i:i + 1].view(np.uint16), yi.view(np.uint16))


def test_torch_port_matches_golden(case):
    """The torch-CPU port (the timed CPU baseline) reproduces the reference's
    unpacked delta bit for bit and its layer output within accumulation noise."""
    import torch
    from oracle import torch_port as T
    bits = int(case["bits"])
    dt = T.dequantize(torch.from_numpy(case["qweight"]), torch.from_numpy(case["qzeros"]),
                      torch.from_numpy(case["scales"]), bits)
    np.testing.assert_array_equal(dt.t().contiguous().numpy().view(np.uint16),
                                  case["dense"].view(np.uint16))
    x = torch.from_numpy(case["x"])
    idx = torch.zeros(x.shape[0], dtype=torch.int64)
    idx[0] = -1
    y = T.apply_delta(x, torch.from_numpy(case["w_base"]),
                      [(torch.from_numpy(case["qweight"]), torch.from_numpy(case["qzeros"]),
                        torch.from_numpy(case["scales"]), bits)], idx).numpy()
    ref = (case["y_base"].astype(np.float32) + case["y_delta"].astype(np.float32))
    ref[0] = case["y_base"][0]
    assert O.rel_l2(y, ref) <= 3e-3


def test_staged_reference_code_agrees_with_the_restatements():
    """Where the reference's own files are staged (oracle/_ref, made by oracle/make_ref.py), its
    QuantLinear.forward / unpack driven by oracle/reference_path.py give what the numpy and
    torch restatements give on the same GPTQ tensors."""
    import torch
    from oracle import deltazip_oracle as orc
    from oracle import reference_path as R
    from oracle import torch_port as T
    if not R.available():
        pytest.skip("reference files not staged on this machine")
    for bits in (2, 4):
        w, deltas = orc.make_layer(256, 384, 3, bits, seed=bits)
        x, idx = orc.make_tokens(21, 384, 3, seed=bits, base_frac=0.2)
        layers = [R.quant_linear(torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc), b)
                  for qw, qz, sc, b in deltas]
        y = R.apply_delta(torch.from_numpy(x), torch.from_numpy(w), layers, torch.from_numpy(idx))
        assert orc.rel_l2(y.numpy(), orc.apply_delta(x, w, deltas, idx)) <= 1e-3
        tdeltas = [tuple(torch.from_numpy(t) for t in d[:3]) + (d[3],) for d in deltas]
        y2 = T.apply_delta(torch.from_numpy(x), torch.from_numpy(w), tdeltas, torch.from_numpy(idx))
        assert orc.rel_l2(y.numpy(), y2.numpy()) <= 1e-3
        dense_t = R.unpack_dense_t(layers[0])
        assert (dense_t.t().numpy().view(np.uint16) == orc.unpack(*deltas[0]).view(np.uint16)).all()


@pytest.mark.parametrize("name", ["sparsegpt_b2_n32_k128", "sparsegpt_b4_n32_k256"])
def test_sparsegpt_golden_is_consistent_with_the_oracle_pieces(name, golden_dir):
    """The compressor's golden vectors (the reference's fasterprune): the grid stored there is the
    oracle's grid of the delta, every value lies on that grid, and every group of four keeps at
    most two non-zero entries."""
    g = np.load(os.path.join(golden_dir, name + ".npz"))
    bits = int(g["bits"])
    scale, zero, maxq = O.find_params_sym(g["delta"], bits)
    np.testing.assert_array_equal(scale, g["scale"])
    np.testing.assert_array_equal(zero, g["zero"])
    codes = g["wq"] / scale[:, None] + zero[:, None]
    assert np.abs(codes - np.rint(codes)).max() < 1e-3 and codes.min() > -0.5 and codes.max() < maxq + 0.5
    assert ((g["wq"] != 0).reshape(g["wq"].shape[0], -1, 4).sum(-1) <= 2).all()
