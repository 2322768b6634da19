"""Tensor-level operators over the C ABI.

`apply_delta` keeps the signature of the reference's op
(serving/vllm/delta/deltazip_marlin.py:10-19):

    y = apply_delta(x, qweight_stacked, scales_stacked, meta_stacked, indices, base_weight)

All tensors are CUDA tensors; work is enqueued on torch's current stream.
PyTorch is used for memory and streams only -- every computation below runs in
libdeltazip_b200.so, with one exception: for prefill-sized batches (more than
FUSED_MAX_TOKENS rows) the plain dense product x W^T, the reference's F.linear
(serving/vllm/model_executor/layers/linear.py:85-96), goes to the library GEMM
(torch.matmul) once, and the library's kernel then adds the delta products into
that result token block by token block.  The fused kernel streams W once per
block of 128 tokens, which is the right trade for decode batches and the wrong
one for thousands of prompt tokens.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import SbmmArgs, check, lib


# Largest batch (rows of x) that takes the fused kernel for base and delta products together.
FUSED_MAX_TOKENS = 512
# In a prefill-sized, sorted batch whose host-side run list is known (Segments.host_runs), a slot
# with at least this many consecutive rows is dequantised once (dz_unpack) and multiplied by the
# library GEMM, as the reference's PyTorch path does (deltazip/nn_modules/qlinear.py:266-330);
# the SBMM kernel would expand the slot's codes once per 32-row window instead.
DENSE_RUN_TOKENS = 256


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("deltazip_b200 operators take CUDA tensors only (no CPU path)")


# ---------------------------------------------------------------------------
# slot format
# ---------------------------------------------------------------------------

def slot_shapes(n: int, k: int, bits: int) -> Tuple[Tuple[int, int], Tuple[int, int], Tuple[int, int]]:
    """(qweight int32, meta int16, scales fp16) shapes of one slot of a [n, k] layer.

    Same outer shapes as the reference's stacked tensors
    (serving/vllm/delta/layers_marlin.py:311-333) for 4-bit; for 2-bit the
    metadata keeps k/16 int16 per row (the reference formula would give k/32,
    which cannot hold two 2-bit positions per group of four)."""
    return (k * bits // 128, 2 * n), (n, k // 16), (1, n)


def alloc_slots(num_slots: int, n: int, k: int, bits: int, device) -> Tuple[torch.Tensor, ...]:
    qs, ms, ss = slot_shapes(n, k, bits)
    return (torch.zeros((num_slots, *qs), dtype=torch.int32, device=device),
            torch.zeros((num_slots, *ms), dtype=torch.int16, device=device),
            torch.zeros((num_slots, *ss), dtype=torch.float16, device=device))


def convert_from_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, bits: int,
                      out: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                      check_status: bool = True):
    """GPTQ-layout tensors of one delta layer -> (qweight, meta, scales) in slot layout."""
    _need_cuda(qweight, qzeros, scales)
    k = qweight.shape[0] * 32 // bits
    n = qweight.shape[1]
    qweight = qweight.contiguous()
    qzeros = qzeros.contiguous()
    scales = scales.contiguous()
    if out is None:
        qs, ms, ss = slot_shapes(n, k, bits)
        out = (torch.empty(qs, dtype=torch.int32, device=qweight.device),
               torch.empty(ms, dtype=torch.int16, device=qweight.device),
               torch.empty(ss, dtype=torch.float16, device=qweight.device))
    sq, sm, ss_ = out
    status = torch.zeros(1, dtype=torch.int32, device=qweight.device)
    check(lib().dz_convert_from_gptq(qweight.data_ptr(), qzeros.data_ptr(), scales.data_ptr(),
                                     n, k, bits, sq.data_ptr(), sm.data_ptr(), ss_.data_ptr(),
                                     status.data_ptr(), _stream()), "dz_convert_from_gptq")
    if check_status:
        host = ctypes.c_int(0)
        check(lib().dz_read_status(status.data_ptr(), _stream(), ctypes.byref(host)), "dz_read_status")
        check(host.value, "dz_convert_from_gptq(device)")
    return out


def unpack(slot_qweight: torch.Tensor, slot_meta: torch.Tensor, slot_scales: torch.Tensor,
           n: int, k: int, bits: int) -> torch.Tensor:
    """Dense fp16 delta [n, k] of one slot (bit-identical to QuantLinear.unpack)."""
    _need_cuda(slot_qweight, slot_meta, slot_scales)
    out = torch.empty((n, k), dtype=torch.float16, device=slot_qweight.device)
    check(lib().dz_unpack(slot_qweight.data_ptr(), slot_meta.data_ptr(), slot_scales.data_ptr(),
                          n, k, bits, out.data_ptr(), _stream()), "dz_unpack")
    return out


# ---------------------------------------------------------------------------
# batch metadata
# ---------------------------------------------------------------------------

class Segments:
    """Device-side segment table for one batch (one scheduling step).

    Built from the per-token slot indices (`base_indices` of the reference's
    convert_mapping, serving/vllm/delta/models.py:69-145) and shared by every
    layer of the step."""

    def __init__(self, max_tokens: int, num_slots: int, device):
        self.max_tokens = int(max_tokens)
        self.num_slots = int(num_slots)
        nbytes = lib().dz_segments_bytes(self.max_tokens, self.num_slots)
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.m = 0
        self.sorted = False
        # [(slot, first row, end row)] of a sorted batch when the caller knows it on the host
        # (the slot manager does); None otherwise.  Only prefill-sized batches use it.
        self.host_runs = None

    def build(self, indices: torch.Tensor, sorted_hint: Optional[bool] = None) -> "Segments":
        """Builds the table on the current stream; never synchronises with the host.
        `sorted_hint=True` is the caller's promise that `indices` is non-decreasing (the
        reference's scheduler delivers batches sorted by delta id,
        serving/vllm/core/scheduler.py:101-104): x is then read in place.  Without the
        promise the SBMM first gathers x into sorted order on the device (a plain copy when
        the batch happens to be sorted), so any order is handled."""
        _need_cuda(indices)
        m = indices.numel()
        if m > self.max_tokens:
            raise ValueError(f"{m} tokens exceed the table capacity {self.max_tokens}")
        if indices.dtype == torch.int64:
            dt = _lib.DZ_INDEX_I64
        elif indices.dtype == torch.int32:
            dt = _lib.DZ_INDEX_I32
        else:
            raise ValueError("indices must be int32 or int64")
        indices = indices.contiguous()
        check(lib().dz_build_segments(indices.data_ptr(), dt, m, self.num_slots,
                                      self.buf.data_ptr(), _stream()), "dz_build_segments")
        self.m = m
        self.sorted = bool(sorted_hint)
        self.host_runs = None
        return self

    def is_sorted_on_device(self) -> bool:
        """What the device-side builder found (synchronises; for tests and diagnostics)."""
        return bool(self.header()[3])

    def header(self):
        """(M, num_slots, num_token_blocks, sorted, status, num_windows, num_active) -- syncs."""
        return tuple(self.buf[:32].view(torch.int32)[:7].tolist())


_workspaces = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    """One grow-only scratch buffer per (device, stream).  The SBMM kernel keeps
    split-K partial tiles and tile counters here; calls on one stream are
    ordered, so they can share it."""
    key = (device.index, _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def read_status(device=None) -> int:
    """Reads and clears the status word the SBMM kernel leaves in the current
    stream's workspace (0 = ok, DZ_ERR_TIMEOUT = a bounded device-side wait ran
    out, DZ_ERR_INVALID_ARG = a wrong `tokens_sorted` promise).  Synchronises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspaces.get((device.index, _stream()))
    if ws is None:
        return 0
    host = ctypes.c_int(0)
    check(lib().dz_read_status(ws.data_ptr(), _stream(), ctypes.byref(host)), "dz_read_status")
    return host.value


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _lib.DZ_DTYPE_F16
    if t.dtype == torch.bfloat16:
        return _lib.DZ_DTYPE_BF16
    raise ValueError(f"unsupported activation dtype {t.dtype}")


def _bits_from_shapes(qweight_stacked: torch.Tensor, k: int) -> int:
    # qweight slot is [k * bits / 128, 2n] int32
    return qweight_stacked.shape[-2] * 128 // k


def sbmm(x: torch.Tensor, qweight_stacked: torch.Tensor, scales_stacked: torch.Tensor,
         meta_stacked: torch.Tensor, segments: Segments, base_weight: Optional[torch.Tensor],
         out: Optional[torch.Tensor] = None, bits: Optional[int] = None,
         _entry: str = "dz_sbmm", accumulate: bool = False, stable: bool = False,
         push=None) -> Optional[torch.Tensor]:
    """y = x W^T + x dequant(delta_slot(i))^T with a prebuilt segment table.  With
    `base_weight=None` only the delta products are computed (rows of slot -1 get 0).
    `out` may be a column slice [:, a:a+N] of a wider row-major tensor; with
    `accumulate=True` the result is added to `out` inside the kernel.  `stable=True` is the
    caller's statement that the base weight, the slot stacks and the segment table were not
    written by the operation right before this call on the stream (DZ_SBMM_INPUTS_STABLE): the
    kernel then starts loading them while its predecessor finishes.  After writing any of them
    with a torch op, call `stream_fence()` before relying on it.  With `push` (a target from
    CustomAllreduce.push_target) the output is not written locally at all: every finished tile
    goes to all tensor-parallel ranks' receive slots and `all_reduce_pushed` yields the sum;
    the call then returns None."""
    _need_cuda(x, qweight_stacked, scales_stacked, meta_stacked)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    m, k = x2.shape
    if base_weight is None:
        n = scales_stacked.shape[-1]
    else:
        _need_cuda(base_weight)
        n = base_weight.shape[0]
        if base_weight.shape[1] != k or not base_weight.is_contiguous():
            raise ValueError("base_weight must be a contiguous [N, K] tensor matching x")
    if segments.m != m:
        raise ValueError(f"segment table was built for {segments.m} tokens, x has {m}")
    if bits is None:
        bits = _bits_from_shapes(qweight_stacked, k)
    if base_weight is not None and m > FUSED_MAX_TOKENS and push is None and _entry == "dz_sbmm":
        # prefill-sized batch: the dense product once through the library GEMM, then the
        # delta products added to it in place (not the early-start form: y is the
        # predecessor's output here)
        base = torch.matmul(x2, base_weight.t())
        if out is None:
            out = base
        else:
            o2 = out.reshape(-1, out.shape[-1]) if out.dim() != 2 else out
            if accumulate:
                o2.add_(base)
            else:
                o2.copy_(base)
        runs = segments.host_runs
        if runs is not None and segments.sorted and \
                all(e - s >= DENSE_RUN_TOKENS for slot, s, e in runs if slot >= 0):
            o2 = out.reshape(-1, out.shape[-1]) if out.dim() != 2 else out
            for slot, s, e in runs:
                if slot < 0:
                    continue
                dense = unpack(qweight_stacked[slot], meta_stacked[slot], scales_stacked[slot],
                               n, k, bits)
                o2[s:e].addmm_(x2[s:e], dense.to(x2.dtype).t())
        else:
            sbmm(x2, qweight_stacked, scales_stacked, meta_stacked, segments, None, out=out,
                 bits=bits, accumulate=True)
        return out.reshape(*x.shape[:-1], n) if out.is_contiguous() else out
    if push is not None:
        if accumulate or out is not None or m == 0:
            raise ValueError("a pushed output takes neither `out` nor `accumulate`, and needs rows")
        nbytes = lib().dz_sbmm_workspace_bytes(m, n, k, int(segments.sorted))
        ws = _workspace(x.device, nbytes)
        args = SbmmArgs(
            x=x2.data_ptr(), w_base=base_weight.data_ptr() if base_weight is not None else None,
            qweight=qweight_stacked.data_ptr(), meta=meta_stacked.data_ptr(),
            scales=scales_stacked.data_ptr(), qweight_stride=qweight_stacked.stride(0) * 4,
            meta_stride=meta_stacked.stride(0) * 2, scales_stride=scales_stacked.stride(0) * 2,
            segments=segments.buf.data_ptr(), y=None, M=m, N=n, K=k,
            num_slots=qweight_stacked.shape[0], bits=bits, dtype=_dtype_code(x),
            tokens_sorted=int(segments.sorted),
            flags=_lib.DZ_SBMM_INPUTS_STABLE if stable else 0,
            workspace=ws.data_ptr(), workspace_bytes=ws.numel(), y_stride=0,
            push=ctypes.pointer(push))
        check(getattr(lib(), _entry)(ctypes.byref(args), _stream()), _entry)
        return None
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs the tensor to add to (out)")
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    out2 = out.reshape(-1, out.shape[-1]) if out.dim() != 2 else out
    if out2.shape != (m, n) or out2.stride(1) != 1 or out2.dtype != x.dtype or \
            (m > 1 and out2.stride(0) < n):
        raise ValueError(f"out must be a [{m}, {n}] {x.dtype} tensor with unit column stride")
    if m == 0:
        return out.reshape(*x.shape[:-1], n) if out.is_contiguous() else out
    nbytes = lib().dz_sbmm_workspace_bytes(m, n, k, int(segments.sorted))
    ws = _workspace(x.device, nbytes)
    args = SbmmArgs(
        x=x2.data_ptr(), w_base=base_weight.data_ptr() if base_weight is not None else None,
        qweight=qweight_stacked.data_ptr(), meta=meta_stacked.data_ptr(),
        scales=scales_stacked.data_ptr(),
        qweight_stride=qweight_stacked.stride(0) * 4, meta_stride=meta_stacked.stride(0) * 2,
        scales_stride=scales_stacked.stride(0) * 2,
        segments=segments.buf.data_ptr(), y=out2.data_ptr(),
        M=m, N=n, K=k, num_slots=qweight_stacked.shape[0], bits=bits, dtype=_dtype_code(x),
        tokens_sorted=int(segments.sorted),
        flags=(_lib.DZ_SBMM_ACCUMULATE if accumulate else 0) | (_lib.DZ_SBMM_INPUTS_STABLE if stable else 0),
        workspace=ws.data_ptr(), workspace_bytes=ws.numel(),
        y_stride=max(out2.stride(0), n))
    check(getattr(lib(), _entry)(ctypes.byref(args), _stream()), _entry)
    return out.reshape(*x.shape[:-1], n) if out.is_contiguous() else out


def stream_fence() -> None:
    """Separates earlier writers on the current stream from later `stable=True` SBMM calls."""
    check(lib().dz_stream_fence(_stream()), "dz_stream_fence")


def base_gemm(x: torch.Tensor, base_weight: torch.Tensor,
              out: Optional[torch.Tensor] = None, stable: bool = False) -> torch.Tensor:
    """y = x W^T on the same kernel (every token base-only); the library GEMM for more than
    FUSED_MAX_TOKENS rows."""
    _need_cuda(x, base_weight)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    m, k = x2.shape
    n = base_weight.shape[0]
    if m > FUSED_MAX_TOKENS:
        if out is None:
            return torch.matmul(x2, base_weight.t()).reshape(*x.shape[:-1], n)
        torch.matmul(x2, base_weight.t(), out=out.reshape(m, n))
        return out.reshape(*x.shape[:-1], n)
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    if m == 0:
        return out.reshape(*x.shape[:-1], n)
    ws = _workspace(x.device, lib().dz_sbmm_workspace_bytes(m, n, k, 1))
    args = SbmmArgs(x=x2.data_ptr(), w_base=base_weight.data_ptr(), y=out.data_ptr(),
                    M=m, N=n, K=k, num_slots=0, bits=4, dtype=_dtype_code(x), tokens_sorted=1,
                    flags=_lib.DZ_SBMM_INPUTS_STABLE if stable else 0,
                    workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    check(lib().dz_base_gemm(ctypes.byref(args), _stream()), "dz_base_gemm")
    return out.reshape(*x.shape[:-1], n)


_segment_cache = {}


def _segments_for(indices: torch.Tensor, num_slots: int, device) -> Segments:
    """Segment table of `indices`, rebuilt only when the tensor changed: the key is the
    buffer's address and torch's version counter, which every in-place write through torch
    (the `copy_` of the reference's _set_delta_mapping, serving/vllm/delta/models.py:407-430)
    advances.  The cache keeps the tensor alive, so the address cannot be handed to another
    tensor while the entry exists.  All layers of a step therefore share one build, with no
    host synchronisation: whether the batch is sorted is left to the device (x is gathered
    through the table's permutation, which is the identity for a sorted batch)."""
    indices = indices.reshape(-1)
    m = indices.numel()
    key = (device.index, _stream(), num_slots)
    stamp = (indices.data_ptr(), indices._version, m, indices.dtype)
    ent = _segment_cache.get(key)
    if ent is None or ent[0].max_tokens < m:
        ent = [Segments(max(m, 256), num_slots, device), None, None]
        _segment_cache[key] = ent
    if ent[1] != stamp:
        ent[0].build(indices)
        ent[1] = stamp
        ent[2] = indices
    return ent[0]


def apply_delta(x: torch.Tensor, qweight_stacked: torch.Tensor, scales_stacked: torch.Tensor,
                meta_stacked: torch.Tensor, indices: torch.Tensor,
                base_weight: torch.Tensor) -> torch.Tensor:
    """Drop-in for the reference op (serving/vllm/delta/deltazip_marlin.py:10-19).  Enqueues
    device work only: no host synchronisation and no allocation besides the result, so it can
    sit inside a captured decode step as the reference's op does."""
    seg = _segments_for(indices, qweight_stacked.shape[0], x.device)
    return sbmm(x, qweight_stacked, scales_stacked, meta_stacked, seg, base_weight)


# ---------------------------------------------------------------------------
# the "separate base output" form of the op: y += x dequant(delta)^T in place
# ---------------------------------------------------------------------------

def add_delta(y: torch.Tensor, x: torch.Tensor, qweight: torch.Tensor,
              qzeros: Optional[torch.Tensor], scales: torch.Tensor,
              g_idx: Optional[torch.Tensor], indices: torch.Tensor,
              meta: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place y[i] += x[i] @ dequant(delta[indices[i]])^T, -1 = nothing added: the
    reference's add_delta (serving/vllm/delta/deltazip.py:14-38) on slot-layout stacks
    (`qweight`, `scales`, `meta` as `alloc_slots` makes them; the symmetric zero point and the
    single quantisation group are implicit, so `qzeros` and `g_idx` are accepted and ignored).
    One launch of the SBMM kernel without its base half, adding into y in its epilogue."""
    if meta is None:
        raise ValueError("slot-layout stacks need their 2:4 metadata (meta)")
    x2 = x.reshape(-1, x.shape[-1])
    y2 = y.view(-1, y.shape[-1])
    seg = _segments_for(indices, qweight.shape[0], x.device)
    sbmm(x2, qweight, scales, meta, seg, None, out=y2, accumulate=True)
    return y


def add_delta_slice(y: torch.Tensor, x: torch.Tensor, qweight: torch.Tensor,
                    qzeros: Optional[torch.Tensor], scales: torch.Tensor,
                    g_idx: Optional[torch.Tensor], indices: torch.Tensor, scale: float,
                    y_offset: int, y_slice_size: int, *, buffer: Optional[torch.Tensor] = None,
                    meta: Optional[torch.Tensor] = None) -> torch.Tensor:
    """add_delta into the columns [y_offset, y_offset + y_slice_size) of y
    (serving/vllm/delta/deltazip.py:41-78; `scale` and `buffer` are unused there too).  The
    kernel writes the slice in place through its row stride; `y_offset` must be a multiple
    of 8 elements."""
    if meta is None:
        raise ValueError("slot-layout stacks need their 2:4 metadata (meta)")
    x2 = x.reshape(-1, x.shape[-1])
    y2 = y.view(-1, y.shape[-1])
    if scales.shape[-1] != y_slice_size:
        raise ValueError(f"slice of {y_slice_size} columns, delta stack has {scales.shape[-1]}")
    seg = _segments_for(indices, qweight.shape[0], x.device)
    sbmm(x2, qweight, scales, meta, seg, None, out=y2[:, y_offset:y_offset + y_slice_size],
         accumulate=True)
    return y


def apply_delta_packed_nslice(x: torch.Tensor, qweight_stacked, qzeros_stacked, scales_stacked,
                              g_idx_stacked, indices: torch.Tensor, output: torch.Tensor,
                              output_slices, meta_stacked=None) -> torch.Tensor:
    """Merged layers (q/k/v, gate/up) whose sub-layers keep separate stacks: one add_delta_slice
    per output slice (serving/vllm/delta/deltazip.py:108-153)."""
    if meta_stacked is None:
        raise ValueError("slot-layout stacks need their 2:4 metadata (meta_stacked)")
    x2 = x.reshape(-1, x.shape[-1])
    out2 = output.view(-1, output.shape[-1])
    offset = 0
    for i, width in enumerate(output_slices):
        add_delta_slice(out2, x2, qweight_stacked[i], qzeros_stacked[i] if qzeros_stacked else None,
                        scales_stacked[i], g_idx_stacked[i] if g_idx_stacked else None,
                        indices, 1.0, offset, width, meta=meta_stacked[i])
        offset += width
    return output


# ---------------------------------------------------------------------------
# per-delta embedding / lm_head (full replacement tables, not additive deltas)
# ---------------------------------------------------------------------------

def _index_code(indices: torch.Tensor) -> int:
    if indices.dtype == torch.int64:
        return _lib.DZ_INDEX_I64
    if indices.dtype == torch.int32:
        return _lib.DZ_INDEX_I32
    raise ValueError("indices must be int32 or int64")


def apply_delta_embed(x: torch.Tensor, delta_weights: torch.Tensor, indices: torch.Tensor,
                      base_weight: torch.Tensor) -> torch.Tensor:
    """Embedding lookup with a replacement table per delta (reference:
    serving/vllm/delta/deltazip_marlin.py:56-86).  x: token ids [M]; delta_weights:
    [D, vocab, hidden]; indices: slot per token (-1 = base_weight [vocab, hidden])."""
    _need_cuda(x, delta_weights, indices, base_weight)
    tokens = x.reshape(-1).to(torch.int64).contiguous()
    indices = indices.reshape(-1).contiguous()
    m = tokens.numel()
    vocab, hidden = base_weight.shape
    out = torch.empty((m, hidden), dtype=base_weight.dtype, device=base_weight.device)
    d = delta_weights.shape[0] if delta_weights is not None and delta_weights.numel() else 0
    check(lib().dz_delta_embedding(
        tokens.data_ptr(), indices.data_ptr(), _index_code(indices), m, hidden,
        base_weight.data_ptr(), delta_weights.data_ptr() if d else None,
        delta_weights.stride(0) * delta_weights.element_size() if d else 0, d, vocab,
        out.data_ptr(), None, _stream()), "dz_delta_embedding")
    return out.reshape(*x.shape, hidden)


_gg_ws = {}


def grouped_gemm(x: torch.Tensor, delta_weights: Optional[torch.Tensor], segments: Segments,
                 base_weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[i] = x[i] T^T with T = base_weight [V, K] for rows of slot -1 and delta_weights[slot]
    ([D, V, K], dense) otherwise, in one launch per 128 rows (dz_grouped_gemm)."""
    _need_cuda(x, delta_weights, base_weight)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    m, k = x2.shape
    v = base_weight.shape[0]
    d = delta_weights.shape[0] if delta_weights is not None and delta_weights.numel() else 0
    if d and (not delta_weights.is_contiguous() or tuple(delta_weights.shape[1:]) != (v, k)):
        raise ValueError("delta_weights must be a contiguous [D, V, K] stack matching base_weight")
    if segments.m != m or segments.num_slots != d:
        raise ValueError("segment table does not match the batch / the number of slots")
    if out is None:
        out = torch.empty((m, v), dtype=x.dtype, device=x.device)
    if m == 0:
        return out.reshape(*x.shape[:-1], v)
    need = lib().dz_grouped_gemm_workspace_bytes(m, k, int(segments.sorted))
    key = (x.device.index, _stream())
    ws = _gg_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 4096), dtype=torch.uint8, device=x.device)
        _gg_ws[key] = ws
    check(lib().dz_grouped_gemm(
        x2.data_ptr(), base_weight.data_ptr(), delta_weights.data_ptr() if d else None,
        v * k * 2 if d else 0, segments.buf.data_ptr(), out.data_ptr(), m, v, k, d, _dtype_code(x),
        int(segments.sorted), out.stride(0), ws.data_ptr(), ws.numel(), _stream()), "dz_grouped_gemm")
    return out.reshape(*x.shape[:-1], v)


def apply_delta_uncompressed(x: torch.Tensor, delta_weights: torch.Tensor, indices: torch.Tensor,
                             base_embedding: torch.Tensor) -> torch.Tensor:
    """lm_head with a full replacement matrix per delta: rows with slot d are multiplied by
    delta_weights[d], rows with -1 by base_embedding (reference:
    serving/vllm/delta/deltazip_marlin.py:21-53, a host loop over the distinct ids).  Here one
    grouped launch on the dense tcgen05 GEMM, no host synchronisation; the vocabulary rows must
    be a multiple of 128 (pad the matrices otherwise)."""
    _need_cuda(x, delta_weights, indices, base_embedding)
    d = delta_weights.shape[0] if delta_weights is not None and delta_weights.numel() else 0
    seg = _segments_for(indices, d, x.device)
    return grouped_gemm(x, delta_weights if d else None, seg, base_embedding.contiguous())


# ---------------------------------------------------------------------------
# the steps between the SBMM calls of a decoder layer (decode time)
# ---------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float,
             residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = rmsnorm(x) * weight; with `residual`, first residual += x (in place) and the norm is
    taken of the sum -- the reference's RMSNorm.forward with and without residual
    (serving/vllm/model_executor/layers/layernorm.py:47-66)."""
    _need_cuda(x, weight, residual)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty_like(x2)
    if residual is not None and not residual.is_contiguous():
        raise ValueError("residual must be contiguous (it is updated in place)")
    check(lib().dz_rms_norm(x2.data_ptr(), residual.data_ptr() if residual is not None else None,
                            weight.data_ptr(), out.data_ptr(), x2.shape[0], x2.shape[1], float(eps),
                            _dtype_code(x), _stream()), "dz_rms_norm")
    return out.reshape(x.shape)


def silu_and_mul(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x[..., :I]) * x[..., I:] (serving/vllm/model_executor/layers/activation.py:17-40)."""
    _need_cuda(x)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    inter = x2.shape[1] // 2
    if out is None:
        out = torch.empty((x2.shape[0], inter), dtype=x.dtype, device=x.device)
    check(lib().dz_silu_and_mul(x2.data_ptr(), out.data_ptr(), x2.shape[0], inter, _dtype_code(x),
                                _stream()), "dz_silu_and_mul")
    return out.reshape(*x.shape[:-1], inter)


def rotary_and_cache(qkv: torch.Tensor, positions: torch.Tensor, q_heads: int, kv_heads: int,
                     rope_theta: float, k_cache: Optional[torch.Tensor] = None,
                     v_cache: Optional[torch.Tensor] = None,
                     slot_mapping: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotary embedding in place on the q and k heads of fused qkv rows [M, (q+2kv)*128] and, when
    a cache is given, the write of k / v to cache slot `slot_mapping[token]`."""
    _need_cuda(qkv, positions, k_cache, v_cache, slot_mapping)
    if not qkv.is_contiguous() or positions.dtype != torch.int64:
        raise ValueError("qkv must be contiguous and positions int64")
    m = qkv.numel() // qkv.shape[-1]
    if slot_mapping is not None and slot_mapping.dtype != torch.int64:
        raise ValueError("slot_mapping must be int64")
    check(lib().dz_rotary_and_cache(
        qkv.data_ptr(), positions.data_ptr(),
        slot_mapping.data_ptr() if slot_mapping is not None else None,
        k_cache.data_ptr() if k_cache is not None else None,
        v_cache.data_ptr() if v_cache is not None else None,
        m, q_heads, kv_heads, qkv.shape[-1] // (q_heads + 2 * kv_heads), float(rope_theta),
        _dtype_code(qkv), _stream()), "dz_rotary_and_cache")
    return qkv


_attn_ws = {}


def paged_attention_decode(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           block_tables: torch.Tensor, seq_lens: torch.Tensor, q_heads: int,
                           kv_heads: int, block_size: int, scale: float, splits: int = 1,
                           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query token per sequence (the q part of fused qkv rows [B, (q+2kv)*128]) against the
    paged cache; returns [B, q_heads*128]."""
    _need_cuda(qkv, k_cache, v_cache, block_tables, seq_lens)
    b = qkv.shape[0]
    if block_tables.dtype != torch.int32 or seq_lens.dtype != torch.int32 or not block_tables.is_contiguous():
        raise ValueError("block_tables / seq_lens must be contiguous int32")
    if out is None:
        out = torch.empty((b, q_heads * 128), dtype=qkv.dtype, device=qkv.device)
    ws_ptr, ws_bytes = None, 0
    if splits > 1:
        need = lib().dz_paged_attention_workspace_bytes(b, q_heads, kv_heads, splits)
        key = (qkv.device.index, _stream())
        ws = _attn_ws.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.zeros(need, dtype=torch.uint8, device=qkv.device)
            _attn_ws[key] = ws
        ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
    check(lib().dz_paged_attention_decode(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        block_tables.data_ptr(), block_tables.shape[1], seq_lens.data_ptr(), b, q_heads, kv_heads,
        128, block_size, float(scale), splits, ws_ptr, ws_bytes, _dtype_code(qkv), _stream()),
        "dz_paged_attention_decode")
    return out
