"""Delta linear layers: the reference's plugin interface over the B200 SBMM.

Same classes, method names and argument meaning as
serving/vllm/delta/layers_marlin.py:47-611 (`DeltaMapping`, `BaseLayerWithDelta`
with create_delta_weights / set_delta / reset_delta / set_mapping /
apply_weights / forward, `from_layer`), so that a model runner written for the
reference drives them unchanged.  The base parallel linears the reference takes
from vLLM (serving/vllm/model_executor/layers/linear.py:157-650) are reduced
here to what the delta layers read from them: the sharded fp16 weight and the
parallel flags.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .config import DeltaConfig
from .custom_all_reduce import get_handle as get_custom_ar_handle
from .parallel_state import (get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size,
                             SHARD_UNIT, shard_range, tensor_model_parallel_all_gather,
                             tensor_model_parallel_all_reduce, tensor_model_parallel_gather)

ASYNC_COPY = True


@dataclass
class DeltaMapping:
    """Per-token and per-sampled-token delta ids of one batch (0 / None = base model)."""
    index_mapping: Tuple[int, ...]
    prompt_mapping: Tuple[int, ...]

    def __post_init__(self):
        self.index_mapping = tuple(self.index_mapping)
        self.prompt_mapping = tuple(self.prompt_mapping)


# ---------------------------------------------------------------------------
# base layers (what the delta layers need of vLLM's parallel linears)
# ---------------------------------------------------------------------------

class _ParallelLinearBase(nn.Module):
    def __init__(self, weight: torch.Tensor):
        super().__init__()
        self.weight = nn.Parameter(weight, requires_grad=False)
        self.bias = None
        self.skip_bias_add = False
        self.tp_size = get_tensor_model_parallel_world_size()

    @property
    def linear_weights(self):
        return {"weight": self.weight}


class ColumnParallelLinear(_ParallelLinearBase):
    """y = x W^T with W split along the output dimension (whole 128-row tiles per rank)."""

    def __init__(self, input_size: int, output_size: int, full_weight: Optional[torch.Tensor] = None,
                 gather_output: bool = False, device="cuda", dtype=torch.float16):
        rank, size = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
        lo, hi = shard_range(output_size, SHARD_UNIT, rank, size)
        if full_weight is None:
            w = torch.empty((hi - lo, input_size), dtype=dtype, device=device).normal_(0, 0.02)
        else:
            w = full_weight[lo:hi].to(device=device, dtype=dtype).contiguous()
        super().__init__(w)
        self.input_size, self.output_size = input_size, output_size
        self.shard = (lo, hi)
        self.gather_output = gather_output

    def forward(self, x):
        y = ops.base_gemm(x, self.weight, stable=True)       # base weights are static
        return (tensor_model_parallel_all_gather(y) if self.gather_output else y), None


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several equally sharded column-parallel matrices stacked (gate_proj + up_proj)."""

    def __init__(self, input_size: int, output_sizes: List[int],
                 full_weights: Optional[List[torch.Tensor]] = None, device="cuda",
                 dtype=torch.float16):
        rank, size = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
        parts, self.shards = [], []
        for i, out in enumerate(output_sizes):
            lo, hi = shard_range(out, SHARD_UNIT, rank, size)
            self.shards.append((lo, hi))
            if full_weights is None:
                parts.append(torch.empty((hi - lo, input_size), dtype=dtype, device=device).normal_(0, 0.02))
            else:
                parts.append(full_weights[i][lo:hi].to(device=device, dtype=dtype))
        _ParallelLinearBase.__init__(self, torch.cat(parts, dim=0).contiguous())
        self.input_size, self.output_sizes = input_size, list(output_sizes)
        self.output_size = sum(output_sizes)
        self.gather_output = False


class QKVParallelLinear(MergedColumnParallelLinear):
    """q, k, v projections stacked; heads are split over the ranks."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: Optional[int] = None,
                 full_weights: Optional[List[torch.Tensor]] = None, device="cuda",
                 dtype=torch.float16):
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        size = get_tensor_model_parallel_world_size()
        self.head_size = head_size
        self.num_heads = total_num_heads // size
        self.num_kv_heads = max(1, total_num_kv_heads // size)
        super().__init__(hidden_size, [total_num_heads * head_size, total_num_kv_heads * head_size,
                                       total_num_kv_heads * head_size], full_weights, device, dtype)


class RowParallelLinear(_ParallelLinearBase):
    """y = x W^T with W split along the input dimension at the same 128-wide boundaries as the
    column-parallel layer that produces x, partial results summed over the ranks."""

    def __init__(self, input_size: int, output_size: int, full_weight: Optional[torch.Tensor] = None,
                 input_is_parallel: bool = True, reduce_results: bool = True, device="cuda",
                 dtype=torch.float16):
        rank, size = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
        lo, hi = shard_range(input_size, SHARD_UNIT, rank, size)
        if full_weight is None:
            w = torch.empty((output_size, hi - lo), dtype=dtype, device=device).normal_(0, 0.02)
        else:
            w = full_weight[:, lo:hi].to(device=device, dtype=dtype).contiguous()
        super().__init__(w)
        self.input_size, self.output_size = input_size, output_size
        self.shard = (lo, hi)
        self.input_is_parallel = input_is_parallel
        self.reduce_results = reduce_results

    def forward(self, x):
        if not self.input_is_parallel:
            x = x[..., self.shard[0]:self.shard[1]].contiguous()
        y = ops.base_gemm(x, self.weight, stable=True)
        if self.reduce_results and self.tp_size > 1:
            y = tensor_model_parallel_all_reduce(y)
        return y, None


# ---------------------------------------------------------------------------
# delta layers
# ---------------------------------------------------------------------------

class BaseLayerWithDelta(nn.Module):
    """Owns the stacked slot tensors of one linear layer and applies the SBMM."""

    def __init__(self, base_layer: nn.Module) -> None:
        super().__init__()
        self.base_layer = base_layer
        self.tp_size = get_tensor_model_parallel_world_size()
        self.tp_rank = get_tensor_model_parallel_rank()
        self.indices: Optional[torch.Tensor] = None
        self.indices_len: Optional[List[int]] = None
        self.segments: Optional[ops.Segments] = None
        self.bits = 4

    # -- slots ---------------------------------------------------------------
    def create_delta_weights(self, max_deltas: int, delta_config: DeltaConfig,
                             model_config=None, storage=None) -> None:
        """Slot stacks of this rank's weight shard [N, K]: qweight int32 [D, K*b/128, 2N], scales
        fp16 [D, 1, N], meta int16 [D, N, K/16].  Allocated (zeroed) here, or taken from
        `storage` = (qweight, meta, scales) when a manager carves them out of its slot arena
        (slots may then be any number of bytes apart; the kernel takes the strides)."""
        n, k = self.base_layer.weight.shape
        self.bits = delta_config.max_bitwidth
        self.pack_factor = delta_config.pack_factor
        self.bitwidth = [0] * max_deltas
        if storage is None:
            storage = ops.alloc_slots(max_deltas, n, k, self.bits, self.base_layer.weight.device)
        else:
            want = ops.slot_shapes(n, k, self.bits)
            for t, shape in zip(storage, want):
                if tuple(t.shape) != (max_deltas, *shape):
                    raise ValueError(f"slot storage {tuple(t.shape)} does not match {(max_deltas, *shape)}")
        self.qweight_stacked, self.meta_stacked, self.scales_stacked = storage

    def reset_delta(self, index: int):
        self.bitwidth[index] = 0
        self.qweight_stacked[index] = 0
        self.scales_stacked[index] = 0
        self.meta_stacked[index] = 0
        ops.stream_fence()        # slot writers never directly precede a forward pass's SBMM

    def set_delta(self, index: int, bitwidth: int, qweight: torch.Tensor,
                  qzeros: Optional[torch.Tensor], scales: torch.Tensor,
                  g_idx: Optional[torch.Tensor] = None, meta: Optional[torch.Tensor] = None):
        """Overwrites slot `index`.  With `meta` the tensors are already in slot layout and are
        copied (asynchronously when they are pinned); with `qzeros` they are GPTQ-layout
        tensors of this rank's shard and are converted on the device."""
        if bitwidth != self.bits:
            raise ValueError(f"slot stack holds {self.bits}-bit deltas, got {bitwidth}")
        self.bitwidth[index] = bitwidth
        if meta is not None:
            self.qweight_stacked[index].copy_(qweight, non_blocking=ASYNC_COPY)
            self.scales_stacked[index].copy_(scales.reshape(self.scales_stacked[index].shape),
                                             non_blocking=ASYNC_COPY)
            self.meta_stacked[index].copy_(meta, non_blocking=ASYNC_COPY)
            ops.stream_fence()
        else:
            dev = self.qweight_stacked.device
            ops.convert_from_gptq(qweight.to(dev, non_blocking=True), qzeros.to(dev, non_blocking=True),
                                  scales.to(dev, non_blocking=True), bitwidth,
                                  out=(self.qweight_stacked[index], self.meta_stacked[index],
                                       self.scales_stacked[index]))

    # -- mapping -------------------------------------------------------------
    def set_mapping(self, base_indices: torch.Tensor, sampler_indices: torch.Tensor = None,
                    sampler_indices_padded: torch.Tensor = None,
                    embeddings_indices: torch.Tensor = None, indices_len: List[int] = None,
                    segments: Optional[ops.Segments] = None):
        """Keeps references to the manager's shared index buffers (and its segment table)."""
        self.indices = base_indices
        self.indices_len = indices_len
        self.segments = segments

    # -- compute -------------------------------------------------------------
    def apply_weights(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if bias is not None:
            raise ValueError("bias is not supported by the delta layers")
        w = self.base_layer.linear_weights["weight"]
        if self.segments is not None:
            # weights are static, slots change only through set_delta / reset_delta / the
            # manager's uploads (all followed by a fence or an event wait) and the table is
            # built by dz_build_segments: the early-start form of the kernel applies
            return ops.sbmm(x, self.qweight_stacked, self.scales_stacked, self.meta_stacked,
                            self.segments, w, out=out, bits=self.bits, stable=True)
        y = ops.apply_delta(x, self.qweight_stacked, self.scales_stacked, self.meta_stacked,
                            self.indices[: self.indices_len[0]], w)
        if out is not None:
            out.copy_(y.reshape(out.shape))
            return out
        return y

    @property
    def linear_weights(self):
        return self.base_layer.linear_weights

    @property
    def weight(self):
        return self.base_layer.weight


class ColumnParallelLinearWithDelta(BaseLayerWithDelta):
    def forward(self, x: torch.Tensor):
        bias = self.base_layer.bias if not self.base_layer.skip_bias_add else None
        out = self.apply_weights(x, bias)
        if getattr(self.base_layer, "gather_output", False):
            out = tensor_model_parallel_all_gather(out)
        return out, (self.base_layer.bias if self.base_layer.skip_bias_add else None)

    @classmethod
    def can_replace_layer(cls, source_layer, delta_config, packed_modules_list, model_config=None):
        return type(source_layer) is ColumnParallelLinear or (
            type(source_layer) is MergedColumnParallelLinear and len(packed_modules_list) == 1)


class MergedColumnParallelLinearWithDelta(ColumnParallelLinearWithDelta):
    """gate_proj + up_proj: one delta tensor set covers both slices (the checkpoint stores the
    merged, per-rank pre-sharded matrix, as the reference's converter writes it)."""

    def create_delta_weights(self, max_deltas, delta_config, model_config=None, storage=None):
        sizes = self.base_layer.output_sizes
        if not (len(sizes) == 2 and sizes[0] == sizes[1]):
            raise ValueError("a merged gate/up delta layer needs two output slices of equal width")
        super().create_delta_weights(max_deltas, delta_config, model_config, storage)

    @classmethod
    def can_replace_layer(cls, source_layer, delta_config, packed_modules_list, model_config=None):
        return type(source_layer) is MergedColumnParallelLinear and len(packed_modules_list) == 2


class MergedQKVParallelLinearWithDelta(ColumnParallelLinearWithDelta):
    def create_delta_weights(self, max_deltas, delta_config, model_config=None, storage=None):
        self.q_proj_shard_size = self.base_layer.num_heads * self.base_layer.head_size
        self.kv_proj_shard_size = self.base_layer.num_kv_heads * self.base_layer.head_size
        super().create_delta_weights(max_deltas, delta_config, model_config, storage)

    @classmethod
    def can_replace_layer(cls, source_layer, delta_config, packed_modules_list, model_config=None):
        return type(source_layer) is QKVParallelLinear and len(packed_modules_list) == 3


class RowParallelLinearWithDelta(BaseLayerWithDelta):
    # True: the SBMM epilogue pushes finished tiles into every rank's receive slot and the
    # reduction sums local memory.  Off by default: measured on 2 and 4 B200s the W-fold 2-byte
    # remote stores lengthen the kernel's tail by more than the pull they replace (N=4: 5.08 ms
    # per step against 4.47 ms with the separate one-shot kernel).
    FUSED_ALL_REDUCE = False

    def forward(self, input_):
        base = self.base_layer
        if base.input_is_parallel:
            x = input_
        else:
            x = input_[..., base.shard[0]:base.shard[1]].contiguous()
        reduce = base.reduce_results and base.tp_size > 1
        if not reduce:
            return self.apply_weights(x), None
        handle = get_custom_ar_handle()
        rows = x.numel() // x.shape[-1]
        n = base.linear_weights["weight"].shape[0]
        if handle is not None and self.FUSED_ALL_REDUCE and self.segments is not None and rows > 0 \
                and handle.can_push(rows, n, x.dtype):
            # fused: the kernel's epilogue stores every finished tile into all ranks' receive
            # slots and flags it; the reduction only sums local memory
            target = handle.push_target(rows, n, x.dtype)
            ops.sbmm(x, self.qweight_stacked, self.scales_stacked, self.meta_stacked, self.segments,
                     base.linear_weights["weight"], bits=self.bits, stable=True, push=target)
            out = handle.all_reduce_pushed(rows, n, x.dtype)
            return out.reshape(*x.shape[:-1], n), None
        staged = None
        nbytes = rows * n * x.element_size()
        if handle is not None and 0 < nbytes <= handle.max_size and nbytes % 16 == 0:
            # produce the partial output directly in peer-visible memory when the
            # peer-memory all-reduce will take it (saves its copy-in)
            staged = handle.staging_like((rows, n), x.dtype)
        out = self.apply_weights(x, out=staged)
        out = tensor_model_parallel_all_reduce(out)
        return out.reshape(*x.shape[:-1], out.shape[-1]), None

    @classmethod
    def can_replace_layer(cls, source_layer, delta_config, packed_modules_list, model_config=None):
        return type(source_layer) is RowParallelLinear


# ---------------------------------------------------------------------------
# embedding and output matrix: a full replacement matrix per delta
# ---------------------------------------------------------------------------

class VocabParallelEmbedding(nn.Module):
    """Token embedding with the vocabulary rows split over the ranks at 128-row units (what the
    delta layer reads of serving/vllm/model_executor/layers/vocab_parallel_embedding.py:47-113)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, full_weight: Optional[torch.Tensor] = None,
                 device="cuda", dtype=torch.float16):
        super().__init__()
        rank, size = get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
        self.org_vocab_size = self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.tp_size = size
        unit = SHARD_UNIT if num_embeddings % SHARD_UNIT == 0 else 1
        self.vocab_start_index, self.vocab_end_index = shard_range(num_embeddings, unit, rank, size)
        self.shard_sizes = [hi - lo for lo, hi in (shard_range(num_embeddings, unit, r, size)
                                                   for r in range(size))]
        rows = self.vocab_end_index - self.vocab_start_index
        if full_weight is None:
            w = torch.empty((rows, embedding_dim), dtype=dtype, device=device).normal_(0, 1.0)
        else:
            w = full_weight[self.vocab_start_index:self.vocab_end_index].to(device=device, dtype=dtype).contiguous()
        self.weight = nn.Parameter(w, requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return self.weight[x]
        outside = (x < self.vocab_start_index) | (x >= self.vocab_end_index)
        local = (x - self.vocab_start_index).masked_fill(outside, 0)
        out = self.weight[local]
        out[outside] = 0
        return tensor_model_parallel_all_reduce(out)


class ParallelLMHead(VocabParallelEmbedding):
    """Output matrix, vocabulary-parallel; its weight is handed to the logits processor."""


class LogitsProcessor(nn.Module):
    """hidden states -> logits over the whole vocabulary on rank 0 (None elsewhere), scaled: what
    the delta layer needs of serving/vllm/model_executor/layers/logits_processor.py:14-84."""

    def __init__(self, vocab_size: int, org_vocab_size: Optional[int] = None, scale: float = 1.0,
                 logits_as_input: bool = False):
        super().__init__()
        self.vocab_size, self.org_vocab_size = vocab_size, org_vocab_size or vocab_size
        self.scale, self.logits_as_input = scale, logits_as_input
        self.include_gpu_probs_tensor = False
        self.shard_sizes: Optional[list] = None

    def forward(self, embedding: torch.Tensor, hidden_states: torch.Tensor,
                embedding_bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        logits = hidden_states if self.logits_as_input else \
            self._get_logits(hidden_states, embedding, embedding_bias)
        if logits is not None:
            logits = logits[..., : self.org_vocab_size]
            if self.scale != 1.0:
                logits = logits * self.scale
        return logits

    def _get_logits(self, hidden_states, embedding, embedding_bias=None):
        logits = ops.base_gemm(hidden_states, embedding) if embedding.shape[0] % 128 == 0 \
            else hidden_states @ embedding.t()
        if embedding_bias is not None:
            logits = logits + embedding_bias
        return tensor_model_parallel_gather(logits, sizes=self.shard_sizes)


class VocabParallelEmbeddingWithDelta(nn.Module):
    """Embedding with a replacement table per delta (serving/vllm/delta/layers_marlin.py:97-171):
    a token of slot d reads delta_weights[d], a base-model token the base table; under tensor
    parallelism every rank looks up the ids of its own vocabulary rows and the rows are summed."""

    def __init__(self, base_layer: VocabParallelEmbedding) -> None:
        super().__init__()
        self.base_layer = base_layer
        self.tp_size = get_tensor_model_parallel_world_size()
        self.tp_rank = get_tensor_model_parallel_rank()
        self.vocab_start_index = base_layer.vocab_start_index
        self.vocab_end_index = base_layer.vocab_end_index
        self.indices = self.embeddings_indices = self.indices_len = None

    def create_delta_weights(self, max_deltas: int, delta_config: DeltaConfig, model_config=None) -> None:
        w = self.base_layer.weight
        self.delta_weights = torch.zeros((max_deltas, *w.shape), dtype=w.dtype, device=w.device)
        self.bitwidth = [0] * max_deltas

    def reset_delta(self, index: int):
        self.bitwidth[index] = 0
        self.delta_weights[index] = 0

    def set_delta(self, index: int, bitwidth: int, weight: torch.Tensor):
        """`weight`: this rank's rows of the delta's table (the reference's per-rank files)."""
        self.bitwidth[index] = bitwidth
        self.delta_weights[index].copy_(weight, non_blocking=ASYNC_COPY)
        ops.stream_fence()

    def set_mapping(self, base_indices, sampler_indices=None, sampler_indices_padded=None,
                    embeddings_indices=None, indices_len=None, segments=None):
        self.indices, self.embeddings_indices, self.indices_len = base_indices, embeddings_indices, indices_len

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        indices = self.indices[: self.indices_len[0]]
        if self.tp_size > 1:
            outside = (x < self.vocab_start_index) | (x >= self.vocab_end_index)
            local = (x - self.vocab_start_index).masked_fill(outside, 0)
        else:
            local = x
        out = ops.apply_delta_embed(local, self.delta_weights, indices, self.base_layer.weight)
        if self.tp_size > 1:
            out[outside] = 0
            out = tensor_model_parallel_all_reduce(out)
        return out

    @classmethod
    def can_replace_layer(cls, source_layer, delta_config, packed_modules_list, model_config=None):
        return type(source_layer) is VocabParallelEmbedding


class LogitsProcessorWithDelta(nn.Module):
    """Logits with a replacement output matrix per delta (layers_marlin.py:614-726): the rows of
    a sequence of slot d are multiplied by weight_stacked[d], base-model rows by the base
    matrix -- one grouped launch (ops.apply_delta_uncompressed) -- and the vocabulary shards are
    gathered on rank 0."""

    def __init__(self, base_layer: LogitsProcessor, hidden_size: int, dtype: torch.dtype, device) -> None:
        super().__init__()
        self.base_layer = base_layer
        self.hidden_size, self.dtype, self.device = hidden_size, dtype, device
        self.tp_size = get_tensor_model_parallel_world_size()
        self.tp_rank = get_tensor_model_parallel_rank()
        self.indices = self.indices_padded = self.indices_len = None
        self.rows: Optional[int] = None

    logits_as_input = property(lambda self: self.base_layer.logits_as_input)
    vocab_size = property(lambda self: self.base_layer.vocab_size)
    scale = property(lambda self: self.base_layer.scale)
    org_vocab_size = property(lambda self: self.base_layer.org_vocab_size)
    include_gpu_probs_tensor = property(lambda self: self.base_layer.include_gpu_probs_tensor)
    shard_sizes = property(lambda self: self.base_layer.shard_sizes)

    def create_delta_weights(self, max_deltas: int, delta_config: DeltaConfig, model_config=None) -> None:
        rows = self.rows if self.rows is not None else self.base_layer.vocab_size // self.tp_size
        self.weight_stacked = torch.zeros((max_deltas, rows, self.hidden_size), dtype=self.dtype,
                                          device=self.device)
        self.bitwidth = [0] * max_deltas

    def reset_delta(self, index: int):
        self.weight_stacked[index] = 0
        self.bitwidth[index] = 0

    def set_delta(self, index: int, bitwidth: int, weight: torch.Tensor):
        self.bitwidth[index] = bitwidth
        self.weight_stacked[index].copy_(weight, non_blocking=ASYNC_COPY)
        ops.stream_fence()

    def set_mapping(self, base_indices, sampler_indices=None, sampler_indices_padded=None,
                    embeddings_indices=None, indices_len=None, segments=None):
        self.indices, self.indices_padded, self.indices_len = sampler_indices, sampler_indices_padded, indices_len

    def _get_logits(self, hidden_states, embedding, embedding_bias=None):
        logits = ops.apply_delta_uncompressed(hidden_states, self.weight_stacked,
                                              self.indices[: self.indices_len[1]], embedding)
        return tensor_model_parallel_gather(logits, sizes=self.shard_sizes)

    def forward(self, *args, **kwargs):
        return type(self.base_layer).forward(self, *args, **kwargs)

    @classmethod
    def can_replace_layer(cls, source_layer, delta_config, packed_modules_list, model_config=None):
        return False            # installed through from_layer_logits_processor, like the reference


def from_layer_logits_processor(layer: LogitsProcessor, lm_head: ParallelLMHead, max_deltas: int,
                                delta_config: DeltaConfig, model_config=None) -> LogitsProcessorWithDelta:
    """The logits processor's delta layer, sized after the output matrix it will be used with
    (layers_marlin.py:752-769)."""
    layer.shard_sizes = lm_head.shard_sizes
    ret = LogitsProcessorWithDelta(layer, lm_head.embedding_dim, lm_head.weight.dtype, lm_head.weight.device)
    ret.rows = lm_head.weight.shape[0]
    ret.create_delta_weights(max_deltas, delta_config, model_config)
    return ret


_all_delta_classes = (MergedQKVParallelLinearWithDelta, MergedColumnParallelLinearWithDelta,
                      ColumnParallelLinearWithDelta, RowParallelLinearWithDelta,
                      VocabParallelEmbeddingWithDelta)


def from_layer(layer: nn.Module, max_deltas: int, delta_config: DeltaConfig,
               packed_modules_list: List, model_config=None, allocate: bool = True) -> nn.Module:
    """Wraps `layer` in the matching delta layer and allocates its slots (returns `layer`
    unchanged when no delta class applies).  With `allocate=False` the caller provides the slot
    storage afterwards through create_delta_weights(..., storage=...)."""
    for cls in _all_delta_classes:
        if cls.can_replace_layer(layer, delta_config, packed_modules_list, model_config):
            ret = cls(layer)
            if allocate:
                ret.create_delta_weights(max_deltas, delta_config, model_config)
            return ret
    return layer
