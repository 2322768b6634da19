"""Slot manager of the delta plugin: mapping conversion, GPU slot allocation, LRU, swap-in.

Counterpart of serving/vllm/delta/models.py (convert_mapping :69-145, DeltaModel :154-263,
DeltaModelManager :266-535, LRUCacheDeltaModelManager :549-603) for the SBMM path.  What
differs by design:
  * the per-token slot indices are turned into the kernel's segment table once per
    scheduling step (`ops.Segments`), shared by every layer, as the reference shares its
    index buffers;
  * activate_delta uploads a delta's slot tensors from pinned host memory on a side stream
    (dz_slot_upload) and the compute stream waits on an event, instead of issuing many small
    copies on the compute stream (serving/vllm/delta/layers_marlin.py:342-360).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import ops
from ._lib import check, lib
from .config import CompressionConfig, DeltaConfig
from .layers import BaseLayerWithDelta, DeltaMapping, from_layer


def convert_mapping(mapping: DeltaMapping, delta_index_to_id: List[Optional[int]], max_deltas: int,
                    vocab_size: int, extra_vocab_size: int, device="cuda"):
    """DeltaMapping -> (base_indices, sampler_indices, sampler_indices_padded,
    embeddings_indices, indices_len), the tensors of the reference's convert_mapping.
    A delta id <= 0 (or None) means the base model: slot -1."""
    slot_of_id = {d: i for i, d in enumerate(delta_index_to_id) if d is not None}

    def slot(x):
        if x is None or x <= 0:
            return -1
        if x not in slot_of_id:
            raise ValueError(f"delta {x} is not active")
        return slot_of_id[x]

    delta_indices = [slot(x) for x in mapping.index_mapping]
    prompt_mapping = [slot(x) for x in mapping.prompt_mapping]
    n = len(delta_indices)
    embedding_indices = [d if d >= 0 else 0 for d in delta_indices]
    indices = torch.tensor([list(range(n)), delta_indices, embedding_indices], dtype=torch.long,
                           device=device)
    prompt = torch.tensor(prompt_mapping, dtype=torch.long, device=device)
    embeddings_indices = torch.stack([indices[2] * extra_vocab_size,
                                      indices[2] * (vocab_size + extra_vocab_size)])
    embeddings_indices[embeddings_indices == -1] = max_deltas - 1
    base_indices = indices[1]
    sampler_indices = prompt
    padded = sampler_indices.clone()
    padded[padded == -1] = max_deltas - 1
    padded = torch.arange(0, len(padded), device=device, dtype=torch.long) + padded * len(padded)
    indices_len = (base_indices.shape[-1], sampler_indices.shape[-1], padded.shape[-1],
                   embeddings_indices.shape[-1])
    return base_indices, sampler_indices, padded, embeddings_indices, indices_len


@dataclass
class DeltaLayerWeights:
    """Slot-layout tensors of one module of one delta (pinned host memory once loaded)."""
    module_name: str
    qweight: Optional[torch.Tensor] = None
    scales: Optional[torch.Tensor] = None
    meta: Optional[torch.Tensor] = None
    qzeros: Optional[torch.Tensor] = None      # only for GPTQ-layout sources
    g_idx: Optional[torch.Tensor] = None
    weight: Optional[torch.Tensor] = None      # uncompressed modules
    compress_config: Optional[CompressionConfig] = None

    @property
    def _compressed(self) -> bool:
        return self.qweight is not None

    def pin_memory(self) -> "DeltaLayerWeights":
        for name in ("qweight", "scales", "meta", "qzeros", "weight"):
            t = getattr(self, name)
            if t is not None and not t.is_cuda and not t.is_pinned() and torch.cuda.is_available():
                setattr(self, name, t.pin_memory())
        return self


def shard_gptq_tensors(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, bits: int,
                       parallel: str, tp_rank: int, tp_size: int
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """This rank's shard of one module's GPTQ-layout tensors (qweight int32 [K*bits/32, N],
    qzeros int32 [1, N*bits/32], scales fp16 [1, N]).

    "column": the output features are cut at whole 128-row tiles (qweight columns, scales and
    packed zero points sliced); "row": the input features are cut at whole 64-wide blocks
    (qweight rows sliced; 2:4 groups and the per-output-channel scales are untouched).  The
    same cuts as the base layers (layers.py) and as the reference's per-rank files
    (serving/vllm/delta/models.py:239-258, written by tools/optimize_io.py:9-66)."""
    from .parallel_state import shard_range
    per = 32 // bits
    k = qweight.shape[0] * per
    n = qweight.shape[1]
    if parallel == "column":
        lo, hi = shard_range(n, 128, tp_rank, tp_size)
        return (qweight[:, lo:hi].contiguous(), qzeros[:, lo // per:hi // per].contiguous(),
                scales[:, lo:hi].contiguous())
    if parallel == "row":
        lo, hi = shard_range(k, 64, tp_rank, tp_size)
        return qweight[lo // per:hi // per].contiguous(), qzeros, scales
    raise ValueError(f"unknown parallel mode {parallel!r}")


class DeltaModel:
    """One fine-tuned variant: module name -> DeltaLayerWeights."""

    def __init__(self, delta_model_id: int, bitwidth: int, deltas: Dict[str, DeltaLayerWeights]):
        self.id = delta_model_id
        self.bitwidth = bitwidth
        self.deltas = deltas

    def get_delta(self, module_name: str) -> Optional[DeltaLayerWeights]:
        return self.deltas.get(module_name)

    @classmethod
    def from_gptq_tensors(cls, delta_model_id: int, bits: int,
                          tensors: Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                          device="cuda") -> "DeltaModel":
        """Builds the slot-layout, pinned-host copy of a delta from per-module GPTQ tensors
        (qweight, qzeros, scales) of this rank's shards -- the conversion the reference does
        offline with an external packer (deltazip/utils/converter.py:12-101) runs here on
        the device at load time."""
        deltas = {}
        for name, (qw, qz, sc) in tensors.items():
            sq, sm, ss = ops.convert_from_gptq(qw.to(device), qz.to(device), sc.to(device), bits)
            deltas[name] = DeltaLayerWeights(name, qweight=sq.cpu(), scales=ss.cpu(), meta=sm.cpu(),
                                             compress_config=CompressionConfig(
                                                 bits=bits, prunen=2, prunem=4)).pin_memory()
        return cls(delta_model_id, bits, deltas)

    @classmethod
    def from_checkpoint(cls, path: str, delta_model_id: int, tp_rank: int = 0) -> "DeltaModel":
        """Reads `deltazip-compressed.safetensors` with the reference's key scheme
        "{module}.{tp_rank}.{qweight|scales|meta}" (serving/vllm/delta/models.py:239-258);
        the tensors must be in this library's slot layout (see tools in ops.convert_from_gptq)."""
        import os
        from safetensors import safe_open
        cfg = CompressionConfig.from_pretrained(path)
        deltas = {}
        with safe_open(os.path.join(path, "deltazip-compressed.safetensors"), "pt") as f:
            keys = list(f.keys())
            modules = sorted({k.rsplit(".", 2)[0] for k in keys if k.endswith(".qweight")})
            for m in modules:
                deltas[m] = DeltaLayerWeights(
                    m, qweight=f.get_tensor(f"{m}.{tp_rank}.qweight"),
                    scales=f.get_tensor(f"{m}.{tp_rank}.scales"),
                    meta=f.get_tensor(f"{m}.{tp_rank}.meta"), compress_config=cfg).pin_memory()
        return cls(delta_model_id, cfg.bits, deltas)


class DeltaModelManager:
    """Keeps registered deltas (pinned host) and the GPU slots of every delta layer."""

    def __init__(self, model: torch.nn.Module, max_num_seqs: int, max_num_batched_tokens: int,
                 vocab_size: int, delta_config: DeltaConfig, device="cuda"):
        self.delta_config = delta_config
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = math.ceil(max_num_batched_tokens / 8) * 8
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self.delta_index_to_id: List[Optional[int]] = [None] * self.delta_slots
        self.base_indices = torch.empty(self.max_num_batched_tokens, dtype=torch.long, device=device)
        self.sampler_indices = torch.empty(self.max_num_batched_tokens, dtype=torch.long, device=device)
        self.sampler_indices_padded = torch.empty(self.max_num_batched_tokens, dtype=torch.long,
                                                  device=device)
        self.embeddings_indices = torch.empty(2, self.max_num_batched_tokens, dtype=torch.long,
                                              device=device)
        self.indices_len: List[int] = [0, 0, 0, 0]
        self.segments = ops.Segments(self.max_num_batched_tokens, self.delta_slots, device)
        self.model = model
        self.supported_delta_modules = list(getattr(model, "supported_delta_modules", []))
        self.packed_modules_mapping = dict(getattr(model, "packed_modules_mapping", {}))
        self.modules: Dict[str, BaseLayerWithDelta] = {}
        self._registered_deltas: Dict[int, DeltaModel] = {}
        self._active_deltas: Dict[int, None] = {}
        self._last_mapping = None
        self.copy_stream = torch.cuda.Stream(device=device) if self.device.type == "cuda" else None
        self._loading: Dict[int, int] = {}                 # delta id -> reserved slot (upload in flight)
        self._slot_ready: List[Optional[torch.cuda.Event]] = [None] * self.delta_slots
        self._slot_released: List[Optional[torch.cuda.Event]] = [None] * self.delta_slots
        self._create_delta_modules()
        model.delta_manager = self

    # -- capacities ----------------------------------------------------------
    @property
    def capacity(self) -> int:
        return self.delta_config.max_cpu_deltas

    @property
    def delta_slots(self) -> int:
        return self.delta_config.max_deltas

    def __len__(self) -> int:
        return len(self._registered_deltas)

    # -- module replacement ----------------------------------------------------
    def _create_delta_modules(self):
        for name, module in list(self.model.named_modules()):
            leaf = name.split(".")[-1]
            if leaf not in self.supported_delta_modules:
                continue
            packed = self.packed_modules_mapping.get(leaf, [leaf])
            new = from_layer(module, self.delta_slots, self.delta_config, packed)
            if new is module:
                continue
            parent = self.model
            parts = name.split(".")
            for p in parts[:-1]:
                parent = getattr(parent, p)
            setattr(parent, parts[-1], new)
            self.modules[name] = new
            new.set_mapping(self.base_indices, self.sampler_indices, self.sampler_indices_padded,
                            self.embeddings_indices, self.indices_len, segments=self.segments)

    # -- registry ----------------------------------------------------------------
    def add_delta(self, delta: DeltaModel) -> bool:
        if delta.id in self._registered_deltas:
            return False
        if len(self._registered_deltas) >= self.capacity:
            raise RuntimeError("No free Delta slots.")
        self._registered_deltas[delta.id] = delta
        return True

    def remove_delta(self, delta_id: int) -> bool:
        self.deactivate_delta(delta_id)
        return bool(self._registered_deltas.pop(delta_id, None))

    def list_deltas(self) -> Dict[int, DeltaModel]:
        return dict(self._registered_deltas)

    def get_delta(self, delta_id: int) -> Optional[DeltaModel]:
        return self._registered_deltas.get(delta_id)

    # -- GPU slots ---------------------------------------------------------------
    def _upload(self, delta: DeltaModel, index: int) -> None:
        """Enqueues the upload of `delta` into slot `index` on the copy stream.  The copy only
        waits for the compute work that was enqueued before the slot was last released (an
        event), so it overlaps with whatever the compute stream is running now."""
        L = lib()
        cs = self.copy_stream.cuda_stream
        rel = self._slot_released[index]
        if rel is not None:
            self.copy_stream.wait_event(rel)
        for name, module in self.modules.items():
            d = delta.get_delta(name)
            if d is None or not d._compressed:
                with torch.cuda.stream(self.copy_stream):
                    module.reset_delta(index)
                continue
            if d.compress_config is not None and d.compress_config.bits != module.bits:
                raise ValueError(f"{name}: {d.compress_config.bits}-bit delta in a {module.bits}-bit stack")
            module.bitwidth[index] = delta.bitwidth
            for src, dst in ((d.qweight, module.qweight_stacked[index]),
                             (d.scales, module.scales_stacked[index]),
                             (d.meta, module.meta_stacked[index])):
                nbytes = dst.numel() * dst.element_size()
                if src.numel() * src.element_size() != nbytes:
                    raise ValueError(f"{name}: slot tensor size mismatch")
                if src.is_cuda:
                    with torch.cuda.stream(self.copy_stream):
                        dst.copy_(src.reshape(dst.shape), non_blocking=True)
                else:
                    check(L.dz_slot_upload(dst.data_ptr(), src.data_ptr(), nbytes, 0, cs),
                          "dz_slot_upload")
        ev = torch.cuda.Event()
        ev.record(self.copy_stream)
        self._slot_ready[index] = ev

    def prefetch_delta(self, delta_id: int) -> bool:
        """Starts moving a registered delta into a free GPU slot without making the compute
        stream wait (the reference prefetches only disk -> pinned host,
        serving/vllm/delta/worker_manager.py:324-333; here the host -> device leg overlaps with
        decode as well).  The slot is reserved; activate_delta later publishes it.  Returns
        False when the delta is already on the GPU or no slot is free."""
        if delta_id in self._active_deltas or delta_id in self._loading:
            return False
        index = next((i for i, d in enumerate(self.delta_index_to_id)
                      if d is None and i not in self._loading.values()), None)
        if index is None:
            return False
        self._loading[delta_id] = index
        self._upload(self._registered_deltas[delta_id], index)
        return True

    def activate_delta(self, delta_id: int) -> bool:
        """Makes the delta usable by the next forward pass: uploads it if prefetch_delta has not
        already, and makes the compute stream wait for the upload's event."""
        if delta_id in self._active_deltas:
            return False
        if delta_id not in self._loading:
            index = next((i for i, d in enumerate(self.delta_index_to_id)
                          if d is None and i not in self._loading.values()), None)
            if index is None:
                raise ValueError("No free delta slots")
            self._loading[delta_id] = index
            self._upload(self._registered_deltas[delta_id], index)
        index = self._loading.pop(delta_id)
        self._active_deltas[delta_id] = None
        self.delta_index_to_id[index] = delta_id
        torch.cuda.current_stream(self.device).wait_event(self._slot_ready[index])
        self._last_mapping = None
        return True

    def deactivate_delta(self, delta_id: int) -> bool:
        if delta_id in self._loading:           # a prefetch that is no longer wanted
            index = self._loading.pop(delta_id)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
            self._slot_released[index] = ev
            return True
        if delta_id not in self._active_deltas:
            return False
        try:
            index = self.delta_index_to_id.index(delta_id)
            self.delta_index_to_id[index] = None
            # kernels enqueued so far may still read the slot: a later upload waits for them
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._slot_released[index] = ev
        except ValueError:
            pass
        self._active_deltas.pop(delta_id)
        self._last_mapping = None
        return True

    def remove_all_deltas(self):
        self._registered_deltas.clear()
        self.delta_index_to_id = [None] * self.delta_slots
        self._active_deltas.clear()
        self._loading.clear()
        self._last_mapping = None

    # -- mapping -------------------------------------------------------------------
    def _set_delta_mapping(self, mapping: DeltaMapping) -> None:
        (base, sampler, padded, emb, indices_len) = convert_mapping(
            mapping, self.delta_index_to_id, self.delta_slots + 1, self.vocab_size,
            self.delta_config.delta_extra_vocab_size, device=self.device)
        self.base_indices[: base.shape[0]].copy_(base)
        self.sampler_indices[: sampler.shape[0]].copy_(sampler)
        self.sampler_indices_padded[: padded.shape[0]].copy_(padded)
        self.embeddings_indices[: emb.shape[0], : emb.shape[1]].copy_(emb)
        self.indices_len[:] = indices_len
        # the host already knows the slot order: no device round trip for the sorted hint
        slot_of_id = {d: i for i, d in enumerate(self.delta_index_to_id) if d is not None}
        s = [slot_of_id.get(x, -1) if (x is not None and x > 0) else -1
             for x in mapping.index_mapping]
        is_sorted = all(s[i] <= s[i + 1] for i in range(len(s) - 1))
        self.segments.build(self.base_indices[: base.shape[0]], sorted_hint=is_sorted)

    def set_delta_mapping(self, mapping: DeltaMapping) -> None:
        if self._last_mapping != mapping:
            self._set_delta_mapping(mapping)
        self._last_mapping = mapping


class LRUCacheDeltaModelManager(DeltaModelManager):
    """DeltaModelManager that evicts the least recently used delta, both from the pinned-host
    registry and from the GPU slots (serving/vllm/delta/models.py:549-603)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._registered_deltas = OrderedDict()
        self._active_deltas = OrderedDict()

    def add_delta(self, delta: DeltaModel) -> bool:
        if delta.id in self._registered_deltas:
            self._registered_deltas.move_to_end(delta.id)
            return False
        while len(self._registered_deltas) >= self.capacity:
            old, _ = next(iter(self._registered_deltas.items()))
            self.remove_delta(old)
        self._registered_deltas[delta.id] = delta
        return True

    def activate_delta(self, delta_id: int) -> bool:
        if delta_id in self._active_deltas:
            self._active_deltas.move_to_end(delta_id)
            return False
        if delta_id not in self._loading and \
                len(self._active_deltas) + len(self._loading) >= self.delta_slots:
            old, _ = next(iter(self._active_deltas.items()))
            self.deactivate_delta(old)
        ok = super().activate_delta(delta_id)
        self._registered_deltas.move_to_end(delta_id)
        return ok

    def remove_oldest_delta(self) -> bool:
        if not self._registered_deltas:
            return False
        old, _ = next(iter(self._registered_deltas.items()))
        return self.remove_delta(old)
