"""CPU port of the reference's PyTorch dequantise-then-matmul path, on torch CPU ops.

TEST / BENCHMARK INFRASTRUCTURE ONLY (the timed CPU baseline and a second
checker); the shipped package never imports it.  It restates, with torch
tensor ops on the host, what the reference runs when no fused kernel is used:
  unpack + matmul   deltazip/nn_modules/qlinear.py:266-341
                    (twin: serving/vllm/delta/quant_linears/quant_linear_naive.py:35-83)
  base GEMM         serving/vllm/model_executor/layers/linear.py:85-96
  per-token select  serving/vllm/delta/deltazip.py:24-30 (loop over distinct ids, -1 = base)
It agrees with the numpy oracle (tests/test_oracle_golden.py checks both
against the golden vectors) and, unlike it, uses the host's BLAS threads the
way the reference does, so it is the one that gets timed.
"""
from __future__ import annotations

import torch


def dequantize(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, bits: int) -> torch.Tensor:
    """GPTQ tensors -> delta^T [K, N] fp16 (the dense matrix the reference multiplies by)."""
    maxq = (1 << bits) - 1
    per = 32 // bits
    shifts = torch.arange(0, 32, bits, dtype=torch.int32)
    w = (qweight.unsqueeze(1) >> shifts.view(1, per, 1)) & maxq          # [K/per, per, N]
    w = w.reshape(-1, qweight.shape[1]).to(torch.int8)
    z = ((qzeros.unsqueeze(2) >> shifts.view(1, 1, per)) & maxq).to(torch.int8) + 1
    z = z.reshape(1, -1)
    return scales.reshape(1, -1) * (w - z)                                # fp16 * int8 -> fp16


def apply_delta(x: torch.Tensor, w_base: torch.Tensor, deltas, indices: torch.Tensor,
                dequant_every_call: bool = True, cache=None) -> torch.Tensor:
    """y[i] = x[i] W^T + x[i] delta_{indices[i]}^T on the CPU, fp16 in / fp16 out."""
    y = torch.nn.functional.linear(x, w_base)
    for d in torch.unique(indices).tolist():
        if d < 0:
            continue
        rows = indices == d
        qw, qz, sc, bits = deltas[d]
        if dequant_every_call or cache is None or d not in cache:
            dt = dequantize(qw, qz, sc, bits)
            if cache is not None:
                cache[d] = dt
        else:
            dt = cache[d]
        y[rows] += torch.matmul(x[rows], dt)
    return y
