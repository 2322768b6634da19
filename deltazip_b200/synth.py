"""Seeded synthetic deltas built on the GPU.

`compress_delta_gptq` is the 2:4-prune + symmetric per-channel quantise + GPTQ
pack pipeline of the reference (deltazip/core/sparsegpt.py:123-136 with H = I,
deltazip/core/quant.py:9-86, deltazip/nn_modules/qlinear.py:83-183) written
with torch tensor ops so that benchmark-size layers (hundreds of millions of
weights) are produced in milliseconds instead of the minutes the reference's
per-column Python loop takes.  It is data preparation: the tensors it returns
are the GPTQ-layout inputs of `ops.convert_from_gptq`.
"""
from __future__ import annotations

from typing import Tuple

import torch


def compress_delta_gptq(delta: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """delta: [N, K] float32 CUDA.  Returns (qweight int32 [K*bits/32, N],
    qzeros int32 [1, N*bits/32], scales fp16 [1, N])."""
    assert delta.dtype == torch.float32 and delta.dim() == 2
    n, k = delta.shape
    maxq = (1 << bits) - 1
    per = 32 // bits
    zero_t = torch.zeros(n, device=delta.device)
    xmin = torch.minimum(delta.min(1)[0], zero_t)
    xmax = torch.maximum(delta.max(1)[0], zero_t)
    xmax = torch.maximum(xmin.abs(), xmax)
    xmin = torch.where(xmin < 0, -xmax, xmin)
    dead = (xmin == 0) & (xmax == 0)
    xmin = torch.where(dead, torch.full_like(xmin, -1.0), xmin)
    xmax = torch.where(dead, torch.full_like(xmax, 1.0), xmax)
    # tensor divisor: with a Python scalar the CUDA kernel multiplies by 1/maxq,
    # which rounds differently from the reference's true division
    scale = ((xmax - xmin) / torch.full_like(xmax, float(maxq))).unsqueeze(1)   # [N, 1]
    zero = float((maxq + 1) // 2)

    g = delta.view(n, k // 4, 4)
    keep_idx = torch.topk(g.abs(), 2, dim=2).indices
    keep = torch.zeros_like(g, dtype=torch.bool).scatter_(2, keep_idx, True).view(n, k)
    pruned = torch.where(keep, delta, torch.zeros_like(delta))
    q = torch.clamp(torch.round(pruned / scale) + zero, 0, maxq)
    wq = scale * (q - zero)
    del g, keep, pruned, q

    scales_h = scale.half()
    inty = torch.round((wq + zero * scale) / scales_h.float()).to(torch.int64)   # [N, K]
    del wq
    inty = inty.t().contiguous().view(k // per, per, n)
    shifts = (torch.arange(per, device=delta.device, dtype=torch.int64) * bits).view(1, per, 1)
    qweight = (inty << shifts).sum(dim=1).to(torch.int32)
    z = torch.full((n // per, per), int(zero) - 1, device=delta.device, dtype=torch.int64)
    qzeros = (z << shifts.view(1, per)).sum(dim=1).to(torch.int32).view(1, n // per)
    return qweight, qzeros, scales_h.view(1, n).contiguous()


def random_delta_slots(num_slots: int, n: int, k: int, bits: int, seed: int, device="cuda",
                       std: float = 1e-3):
    """`num_slots` seeded deltas ~ N(0, std) compressed and converted into a slot stack."""
    from . import ops
    gen = torch.Generator(device=device).manual_seed(seed)
    qs, ms, ss = ops.alloc_slots(num_slots, n, k, bits, device)
    for d in range(num_slots):
        delta = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * std
        qw, qz, sc = compress_delta_gptq(delta, bits)
        del delta
        ops.convert_from_gptq(qw, qz, sc, bits, out=(qs[d], ms[d], ss[d]), check_status=(d == 0))
    return qs, ms, ss
