"""The reference's own CPU path for one SBMM call, driven from its staged source files.

TEST / BENCHMARK INFRASTRUCTURE ONLY (the timed CPU baseline and a cross-check of the
restatements in this folder); the shipped package never imports it.

What runs is the reference's code, unmodified, loaded by file path from oracle/_ref/
(see oracle/make_ref.py):
    QuantLinear.forward   deltazip/nn_modules/qlinear.py:266-341  (dequantise, then matmul)
    QuantLinear.unpack    deltazip/nn_modules/qlinear.py:185-264  (dense delta)
Around it, in the few lines below, the two steps the serving code adds:
    base GEMM             F.linear, serving/vllm/model_executor/layers/linear.py:85-96
    per-token selection   loop over the distinct delta ids of the batch, -1 = base only,
                          serving/vllm/delta/deltazip.py:24-30 / deltazip_marlin.py:44-53
"""
from __future__ import annotations

import importlib.util
import os

import torch

_REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
_mods = {}


def available() -> bool:
    return all(os.path.isfile(os.path.join(_REF_DIR, f)) for f in ("quant.py", "qlinear.py"))


def _load(name: str):
    if name not in _mods:
        spec = importlib.util.spec_from_file_location("dz_ref_" + name, os.path.join(_REF_DIR, name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mods[name] = mod
    return _mods[name]


def quant_linear(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, bits: int):
    """A reference QuantLinear holding the given GPTQ tensors (one group: g_idx == 0)."""
    ql = _load("qlinear")
    k = qweight.shape[0] * 32 // bits
    n = qweight.shape[1]
    layer = ql.QuantLinear(bits, k, n, bias=False)
    layer.qweight = qweight
    layer.qzeros = qzeros
    layer.scales = scales
    return layer


def apply_delta(x: torch.Tensor, w_base: torch.Tensor, layers, indices: torch.Tensor,
                pre_unpacked=None) -> torch.Tensor:
    """y[i] = x[i] W^T + QuantLinear_{indices[i]}.forward(x[i]); `pre_unpacked` (list of dense
    fp16 delta^T [K, N] from QuantLinear.unpack) skips the per-call dequantisation."""
    y = torch.nn.functional.linear(x, w_base)
    for d in torch.unique(indices).tolist():
        if d < 0:
            continue
        rows = indices == d
        if pre_unpacked is not None:
            y[rows] += torch.matmul(x[rows], pre_unpacked[d])
        else:
            y[rows] += layers[d].forward(x[rows])
    return y


def unpack_dense_t(layer) -> torch.Tensor:
    """delta^T [K, N] fp16 from the reference's unpack (which returns an nn.Linear [N, K])."""
    return layer.unpack().weight.data.half().t().contiguous()


def quantizer():
    return _load("quant")
