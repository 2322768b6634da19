"""Delta compression on the GPU: 2:4 pruning + symmetric low-bit quantisation with SparseGPT's
error feedback, then packing -- the producer of the tensors the SBMM path serves.

Follows deltazip/core/sparsegpt.py (`SparseGPT.add_batch` :25-43, `fasterprune` :45-196 with
prunen:prunem = 2:4, no activation ordering) and `QuantLinear.pack`
(deltazip/nn_modules/qlinear.py:83-183).  The per-column loop of a block -- mask, quantise,
propagate the error inside the block -- is one kernel launch per 128 columns (dz_sparsegpt_block,
rows in parallel); the dense linear algebra around it (Cholesky factorisations of H, the
rank-128 update of the columns behind a block) are library calls, as in the reference.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ._lib import check, lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class HessianAccumulator:
    """Running H = (2 / n) sum x x^T over calibration inputs of a linear layer (sparsegpt.py:25-43)."""

    def __init__(self, columns: int, device="cuda"):
        self.H = torch.zeros((columns, columns), dtype=torch.float32, device=device)
        self.nsamples = 0

    def add_batch(self, inp: torch.Tensor) -> None:
        if inp.dim() == 2:
            inp = inp.unsqueeze(0)
        batch = inp.shape[0]
        x = inp.reshape(-1, inp.shape[-1]).t().float()
        self.H *= self.nsamples / (self.nsamples + batch)
        self.nsamples += batch
        x = math.sqrt(2 / self.nsamples) * x
        self.H += x.matmul(x.t())


def hinv_factor(H: torch.Tensor, percdamp: float = 0.01) -> Tuple[torch.Tensor, torch.Tensor]:
    """Upper Cholesky factor of the damped H^-1 and the mask of dead columns (sparsegpt.py:69-88)."""
    H = H.clone()
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    damp = percdamp * torch.mean(torch.diag(H))
    idx = torch.arange(H.shape[0], device=H.device)
    H[idx, idx] += damp
    H = torch.linalg.cholesky(H)
    H = torch.cholesky_inverse(H)
    return torch.linalg.cholesky(H, upper=True).contiguous(), dead


def find_params(W: torch.Tensor, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row symmetric grid (scale [N], zero [N]) of W [N, K] float32."""
    n, k = W.shape
    scale = torch.empty(n, dtype=torch.float32, device=W.device)
    zero = torch.empty(n, dtype=torch.float32, device=W.device)
    check(lib().dz_quant_find_params(W.data_ptr(), n, k, bits, scale.data_ptr(), zero.data_ptr(),
                                     _stream()), "dz_quant_find_params")
    return scale, zero


def sparsegpt_2_4(delta: torch.Tensor, bits: int, H: Optional[torch.Tensor] = None,
                  percdamp: float = 0.01, blocksize: int = 128, hinv: Optional[torch.Tensor] = None):
    """2:4-pruned, `bits`-bit quantised delta with SparseGPT error feedback.

    delta: [N, K] float32 CUDA (target weight minus base weight); H: [K, K] Hessian from
    HessianAccumulator (None = identity: no error feedback, the "keep the two largest of four"
    rule); `hinv` supplies the upper Cholesky factor of the damped H^-1 directly.  Returns (Wq float32 [N, K] on the quantisation grid, scale [N], zero [N], loss [N])."""
    if not delta.is_cuda or delta.dtype != torch.float32 or delta.dim() != 2:
        raise ValueError("delta must be a 2-D float32 CUDA tensor")
    if blocksize > 128 or blocksize % 4:
        raise ValueError("blocksize must be a multiple of 4, at most 128")
    n, k = delta.shape
    if k % 4:
        raise ValueError("K must be a multiple of 4")
    W = delta.clone().contiguous()
    scale, zero = find_params(W, bits)
    if hinv is None:
        if H is None:
            H = torch.eye(k, dtype=torch.float32, device=W.device)
        hinv, dead = hinv_factor(H.to(W.device, torch.float32), percdamp)
        W[:, dead] = 0
    else:
        hinv = hinv.to(W.device, torch.float32).contiguous()
    loss = torch.zeros(n, dtype=torch.float32, device=W.device)
    L = lib()
    for i1 in range(0, k, blocksize):
        i2 = min(i1 + blocksize, k)
        count = i2 - i1
        Q = torch.empty((n, count), dtype=torch.float32, device=W.device)
        E = torch.empty((n, count), dtype=torch.float32, device=W.device)
        check(L.dz_sparsegpt_block(W.data_ptr() + 4 * i1, k, hinv.data_ptr() + 4 * (i1 * k + i1), k,
                                   scale.data_ptr(), zero.data_ptr(), bits, n, count, Q.data_ptr(),
                                   E.data_ptr(), loss.data_ptr(), _stream()), "dz_sparsegpt_block")
        W[:, i1:i2] = Q
        if i2 < k:
            W[:, i2:] -= E.matmul(hinv[i1:i2, i2:])
    return W, scale, zero, loss


def pack_gptq(Wq: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, bits: int):
    """(qweight int32 [K*bits/32, N], qzeros int32 [1, N*bits/32], scales fp16 [1, N])."""
    n, k = Wq.shape
    per = 32 // bits
    qweight = torch.empty((k // per, n), dtype=torch.int32, device=Wq.device)
    qzeros = torch.empty((1, n // per), dtype=torch.int32, device=Wq.device)
    scales = torch.empty((1, n), dtype=torch.float16, device=Wq.device)
    check(lib().dz_pack_gptq(Wq.contiguous().data_ptr(), scale.data_ptr(), zero.data_ptr(), n, k, bits,
                             qweight.data_ptr(), qzeros.data_ptr(), scales.data_ptr(), _stream()),
          "dz_pack_gptq")
    return qweight, qzeros, scales


def compress_delta(delta: torch.Tensor, bits: int, H: Optional[torch.Tensor] = None,
                   percdamp: float = 0.01):
    """delta [N, K] float32 -> GPTQ-layout tensors of the compressed delta (and the per-row
    loss); `ops.convert_from_gptq` turns them into slot layout."""
    Wq, scale, zero, loss = sparsegpt_2_4(delta, bits, H, percdamp)
    return pack_gptq(Wq, scale, zero, bits) + (loss,)
