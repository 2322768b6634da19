"""Slot manager of the delta plugin: mapping conversion, delta loading, GPU slot allocation,
LRU, swap-in.

Counterpart of serving/vllm/delta/models.py (convert_mapping :69-145, DeltaModel :154-263,
DeltaModelManager :266-535, LRUCacheDeltaModelManager :549-603) for the SBMM path.  What
differs by design:
  * the per-token slot indices are turned into the kernel's segment table once per
    scheduling step (`ops.Segments`), shared by every layer, as the reference shares its
    index buffers;
  * all slot tensors of one GPU slot (every module's qweight / meta / scales) live in one
    contiguous device arena, and a registered delta keeps the same bytes in one pinned host
    arena, so a swap-in is ONE asynchronous host-to-device copy on a side stream
    (dz_slot_upload) that the compute stream joins through an event, instead of three small
    copies per module on the compute stream (serving/vllm/delta/layers_marlin.py:342-360);
  * deltas written by the reference's compressor in GPTQ layout are converted to the slot
    layout on the device while loading (`DeltaModel.from_reference_checkpoint`).
"""
from __future__ import annotations

import json
import math
import os
import re
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import ops
from ._lib import check, lib
from .config import CompressionConfig, DeltaConfig
from .layers import (BaseLayerWithDelta, DeltaMapping, LogitsProcessor, LogitsProcessorWithDelta,
                     VocabParallelEmbeddingWithDelta, from_layer, from_layer_logits_processor)


def _convert_mapping(mapping: DeltaMapping, delta_index_to_id: List[Optional[int]], max_deltas: int,
                     vocab_size: int, extra_vocab_size: int, device="cuda"):
    """DeltaMapping -> (base_indices, sampler_indices, sampler_indices_padded,
    embeddings_indices, indices_len), the index tensors the reference's convert_mapping
    produces (serving/vllm/delta/models.py:69-145).  A delta id <= 0 (or None) means the base
    model: slot -1.

    The slot of every token comes from one table lookup over the whole batch (the reference
    searches the slot list once per token); the lookup and the "is this delta active" check run
    on the host's copy of the ids, and the five tensors reach the device in one copy, so nothing
    here waits for the GPU.  Also returns (whether the token slots are non-decreasing, and for a
    sorted batch of more than ops.FUSED_MAX_TOKENS rows its runs [(slot, first row, end row)])."""
    ids = torch.tensor([0 if x is None else x for x in mapping.index_mapping], dtype=torch.long)
    prompt_ids = torch.tensor([0 if x is None else x for x in mapping.prompt_mapping], dtype=torch.long)
    active = [d for d in delta_index_to_id if d is not None]
    top = max([int(ids.max()) if ids.numel() else 0, int(prompt_ids.max()) if prompt_ids.numel() else 0]
              + active + [0])
    table = torch.full((top + 2,), -2, dtype=torch.long)      # -2 = not resident
    table[0] = -1
    for slot, d in enumerate(delta_index_to_id):
        if d is not None:
            table[d] = slot
    slots = table[ids.clamp_min(0)]
    prompt_slots = table[prompt_ids.clamp_min(0)]
    missing = torch.cat([ids[slots == -2], prompt_ids[prompt_slots == -2]])
    if missing.numel():
        raise ValueError(f"delta {int(missing[0])} is not active")
    n, s = ids.numel(), prompt_ids.numel()
    # per-token rows: slot, slot clamped at 0 for the embedding offsets
    emb = slots.clamp_min(0)
    packed = torch.empty((4, max(n, s)), dtype=torch.long)
    packed[0, :n] = slots
    packed[1, :n] = emb * extra_vocab_size
    packed[2, :n] = emb * (vocab_size + extra_vocab_size)
    last = max_deltas - 1                                        # where base-model rows point
    pad = torch.where(prompt_slots < 0, torch.full_like(prompt_slots, last), prompt_slots)
    packed[3, :s] = torch.arange(s, dtype=torch.long) + pad * s
    on_dev = packed.to(device, non_blocking=True)
    base_indices = on_dev[0, :n]
    embeddings_indices = on_dev[1:3, :n]
    sampler_indices = prompt_slots.to(device, non_blocking=True)
    sampler_indices_padded = on_dev[3, :s]
    indices_len = (n, s, s, n)
    is_sorted = bool(n < 2 or (slots[1:] >= slots[:-1]).all())
    runs = None
    if is_sorted and n > ops.FUSED_MAX_TOKENS:
        # prefill-sized batch: the runs of equal slots (host side), for the dequantise-once path
        cuts = (torch.nonzero(slots[1:] != slots[:-1]).flatten() + 1).tolist()
        runs = [(int(slots[a]), a, b) for a, b in zip([0] + cuts, cuts + [n])]
    return (base_indices, sampler_indices, sampler_indices_padded, embeddings_indices,
            indices_len), (is_sorted, runs)


def convert_mapping(mapping: DeltaMapping, delta_index_to_id: List[Optional[int]], max_deltas: int,
                    vocab_size: int, extra_vocab_size: int, device="cuda"):
    """Public form with the reference's return value (the five index tensors / lengths)."""
    return _convert_mapping(mapping, delta_index_to_id, max_deltas, vocab_size, extra_vocab_size,
                            device)[0]


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
    packed zero points sliced); "row": the input features are cut at the same 128-wide
    boundaries (qweight rows sliced; 2:4 groups and the per-output-channel scales are
    untouched).  The same cuts as the base layers (layers.py) and as the reference's per-rank files
    (serving/vllm/delta/models.py:239-258, written by tools/optimize_io.py:9-66)."""
    from .parallel_state import SHARD_UNIT, shard_range
    per = 32 // bits
    k = qweight.shape[0] * per
    n = qweight.shape[1]
    if parallel == "column":
        lo, hi = shard_range(n, SHARD_UNIT, tp_rank, tp_size)
        return (qweight[:, lo:hi].contiguous(), qzeros[:, lo // per:hi // per].contiguous(),
                scales[:, lo:hi].contiguous())
    if parallel == "row":
        lo, hi = shard_range(k, SHARD_UNIT, tp_rank, tp_size)
        return qweight[lo // per:hi // per].contiguous(), qzeros, scales
    raise ValueError(f"unknown parallel mode {parallel!r}")


class SlotLayout:
    """Byte offsets of every delta module's qweight / meta / scales inside one slot arena
    (each region 256-byte aligned).  The same layout describes a GPU slot and the pinned host
    copy of a registered delta."""

    def __init__(self):
        self.regions: Dict[str, Tuple[int, int, int, int, int, int]] = {}
        self.total = 0

    def add(self, name: str, n: int, k: int, bits: int) -> None:
        sizes = (n * k * bits // 16, n * k // 8, n * 2)
        offs = []
        for nbytes in sizes:
            offs.append(self.total)
            self.total += (nbytes + 255) // 256 * 256
        self.regions[name] = (offs[0], sizes[0], offs[1], sizes[1], offs[2], sizes[2])


# module names of a reference checkpoint (HuggingFace Llama naming) -> (module of the serving
# model, position inside a merged module)
_REF_KEY = re.compile(r"^(?:model\.)?layers\.(\d+)\.(?:self_attn|mlp)\.(\w+)_proj\.(qweight|qzeros|scales|g_idx)$")
_MERGED = {"q": ("qkv_proj", 0), "k": ("qkv_proj", 1), "v": ("qkv_proj", 2), "o": ("o_proj", 0),
           "gate": ("gate_up_proj", 0), "up": ("gate_up_proj", 1), "down": ("down_proj", 0)}
_ROW_PARALLEL = ("o_proj", "down_proj")


def read_reference_tensors(path: str, tp_rank: int = 0, tp_size: int = 1):
    """Reads a delta as the reference's compressor writes it -- `deltazip-compressed.safetensors`
    holding the QuantLinear buffers of every projection under HuggingFace names
    ("model.layers.3.self_attn.q_proj.qweight", ".qzeros", ".scales", ".g_idx";
    deltazip/modeling/_base.py:597-648) next to `compress_config.json` -- and returns
    (CompressionConfig, {serving module name: (qweight, qzeros, scales)}) for this rank:
    q/k/v and gate/up are cut per projection at the tensor-parallel boundaries and concatenated
    along the output dimension, as the serving model merges them
    (deltazip/utils/converter.py:55-90); o_proj / down_proj are cut along the input dimension
    (serving/vllm/tools/optimize_io.py:9-66).  Host tensors only; no GPU involved.

    Raises FileNotFoundError for a missing file, ValueError for an unservable configuration, a
    missing projection or mismatching shapes; a truncated file surfaces as the safetensors
    reader's error."""
    from safetensors import safe_open
    cfg = CompressionConfig.from_pretrained(path)
    if not cfg.servable():
        raise ValueError(f"{path}: only 2:4-sparse, symmetric, per-channel 2/4-bit deltas are servable "
                         f"(got {cfg.to_dict()})")
    file = os.path.join(path, "deltazip-compressed.safetensors")
    if not os.path.isfile(file):
        raise FileNotFoundError(file)
    parts: Dict[str, Dict[int, Dict[str, torch.Tensor]]] = {}
    with safe_open(file, "pt") as f:
        for key in f.keys():
            m = _REF_KEY.match(key)
            if not m or m.group(2) not in _MERGED:
                continue
            merged, pos = _MERGED[m.group(2)]
            parts.setdefault(f"layers.{m.group(1)}.{merged}", {}).setdefault(pos, {})[m.group(3)] = \
                f.get_tensor(key)
    if not parts:
        raise ValueError(f"{file}: no compressed projection found")
    out = {}
    for name, subs in sorted(parts.items()):
        leaf = name.rsplit(".", 1)[1]
        want = {"qkv_proj": 3, "gate_up_proj": 2}.get(leaf, 1)
        if sorted(subs) != list(range(want)):
            raise ValueError(f"{name}: expected {want} projection(s), found {sorted(subs)}")
        shards = []
        for pos in range(want):
            t = subs[pos]
            for need in ("qweight", "qzeros", "scales"):
                if need not in t:
                    raise ValueError(f"{name}: tensor {need} is missing")
            qw, qz, sc = t["qweight"], t["qzeros"], t["scales"].reshape(1, -1)
            n = qw.shape[1]
            if qw.dtype != torch.int32 or sc.shape[1] != n or qz.numel() * 32 // cfg.bits != n:
                raise ValueError(f"{name}: qweight {tuple(qw.shape)} / qzeros {tuple(qz.shape)} / "
                                 f"scales {tuple(sc.shape)} do not describe one {cfg.bits}-bit layer")
            if "g_idx" in t and int(t["g_idx"].abs().max()) != 0:
                raise ValueError(f"{name}: grouped scales (g_idx != 0) are not servable")
            shards.append(shard_gptq_tensors(qw, qz.reshape(1, -1), sc.half(), cfg.bits,
                                             "row" if leaf in _ROW_PARALLEL else "column",
                                             tp_rank, tp_size))
        if len({s[0].shape[0] for s in shards}) != 1:
            raise ValueError(f"{name}: merged projections disagree on the input width")
        out[name] = (torch.cat([s[0] for s in shards], dim=1).contiguous(),
                     torch.cat([s[1] for s in shards], dim=1).contiguous(),
                     torch.cat([s[2] for s in shards], dim=1).contiguous())
    return cfg, out


class DeltaModel:
    """One fine-tuned variant: module name -> DeltaLayerWeights (slot layout, host memory)."""

    def __init__(self, delta_model_id: int, bitwidth: int, deltas: Dict[str, DeltaLayerWeights]):
        self.id = delta_model_id
        self.bitwidth = bitwidth
        self.deltas = deltas
        self.arena: Optional[torch.Tensor] = None        # pinned uint8 [layout.total] once packed
        self._arena_layout: Optional[SlotLayout] = None

    def get_delta(self, module_name: str) -> Optional[DeltaLayerWeights]:
        return self.deltas.get(module_name)

    def pack(self, layout: SlotLayout) -> torch.Tensor:
        """One pinned host buffer holding this delta's bytes exactly as a GPU slot holds them
        (modules the delta lacks stay zero, which is what a reset slot contains).  The
        per-module tensors become views of the buffer."""
        if self.arena is not None and self._arena_layout is layout:
            return self.arena
        arena = torch.zeros(layout.total, dtype=torch.uint8)
        if torch.cuda.is_available():
            arena = arena.pin_memory()
        for name, (qo, qb, mo, mb, so, sb) in layout.regions.items():
            d = self.deltas.get(name)
            if d is None or not d._compressed:
                continue
            for t, off, nbytes, attr in ((d.qweight, qo, qb, "qweight"), (d.meta, mo, mb, "meta"),
                                         (d.scales, so, sb, "scales")):
                src = t.detach().cpu().contiguous()
                if src.numel() * src.element_size() != nbytes:
                    raise ValueError(f"{name}.{attr}: {src.numel() * src.element_size()} bytes, the "
                                     f"slot holds {nbytes}")
                region = arena[off:off + nbytes]
                region.copy_(src.view(torch.uint8).reshape(-1))
                setattr(d, attr, region.view(src.dtype).reshape(src.shape))
        self.arena, self._arena_layout = arena, layout
        return arena

    @classmethod
    def from_gptq_tensors(cls, delta_model_id: int, bits: int,
                          tensors: Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                          device="cuda") -> "DeltaModel":
        """Builds the slot-layout host copy of a delta from per-module GPTQ tensors
        (qweight, qzeros, scales) of this rank's shards -- the conversion the reference does
        offline with an external packer (deltazip/utils/converter.py:12-101) runs here on
        the device at load time."""
        deltas = {}
        for name, (qw, qz, sc) in tensors.items():
            sq, sm, ss = ops.convert_from_gptq(qw.to(device), qz.to(device), sc.to(device), bits)
            deltas[name] = DeltaLayerWeights(name, qweight=sq.cpu(), scales=ss.cpu(), meta=sm.cpu(),
                                             compress_config=CompressionConfig(
                                                 bits=bits, prunen=2, prunem=4))
        return cls(delta_model_id, bits, deltas)

    @classmethod
    def from_reference_checkpoint(cls, path: str, delta_model_id: int, tp_rank: int = 0,
                                  tp_size: int = 1, device="cuda",
                                  prefetch_thread_event=None, discard_prefetching_event=None
                                  ) -> Optional["DeltaModel"]:
        """Loads a delta written by the reference's compressor (GPTQ layout, HuggingFace module
        names) and converts it to slot layout on the device.  The two events are the
        reference's pause / abort handshake for background loads
        (serving/vllm/delta/models.py:171-232): the load waits while `prefetch_thread_event`
        is cleared and returns None once `discard_prefetching_event` is set."""
        if discard_prefetching_event is not None and discard_prefetching_event.is_set():
            return None
        if prefetch_thread_event is not None:
            prefetch_thread_event.wait()
        cfg, tensors = read_reference_tensors(path, tp_rank, tp_size)
        deltas = {}
        for name, (qw, qz, sc) in tensors.items():
            if discard_prefetching_event is not None and discard_prefetching_event.is_set():
                return None
            if prefetch_thread_event is not None:
                prefetch_thread_event.wait()
            sq, sm, ss = ops.convert_from_gptq(qw.to(device), qz.to(device), sc.to(device), cfg.bits)
            deltas[name] = DeltaLayerWeights(name, qweight=sq.cpu(), scales=ss.cpu(), meta=sm.cpu(),
                                             compress_config=cfg)
        return cls(delta_model_id, cfg.bits, deltas)

    @classmethod
    def from_checkpoint(cls, path: str, delta_model_id: int, tp_rank: int = 0, tp_size: int = 1,
                        device="cuda", prefetch_thread_event=None,
                        discard_prefetching_event=None) -> Optional["DeltaModel"]:
        """Loads a delta directory.  Two contents are understood: the serving key scheme
        "{module}.{tp_rank}.{qweight|scales|meta}" (serving/vllm/delta/models.py:239-258) with
        tensors already in this library's slot layout, and the compressor's GPTQ artefact
        (`from_reference_checkpoint`)."""
        from safetensors import safe_open
        file = os.path.join(path, "deltazip-compressed.safetensors")
        if not os.path.isfile(file):
            raise FileNotFoundError(file)
        with safe_open(file, "pt") as f:
            keys = list(f.keys())
            if not any(k.endswith(f".{tp_rank}.meta") for k in keys):
                return cls.from_reference_checkpoint(path, delta_model_id, tp_rank, tp_size, device,
                                                     prefetch_thread_event, discard_prefetching_event)
            cfg = CompressionConfig.from_pretrained(path)
            deltas = {}
            modules = sorted({k.rsplit(".", 2)[0] for k in keys if k.endswith(".qweight")})
            for m in modules:
                if discard_prefetching_event is not None and discard_prefetching_event.is_set():
                    return None
                if prefetch_thread_event is not None:
                    prefetch_thread_event.wait()
                deltas[m] = DeltaLayerWeights(
                    m, qweight=f.get_tensor(f"{m}.{tp_rank}.qweight"),
                    scales=f.get_tensor(f"{m}.{tp_rank}.scales"),
                    meta=f.get_tensor(f"{m}.{tp_rank}.meta"), compress_config=cfg)
        return cls(delta_model_id, cfg.bits, deltas)

    def save_slot_checkpoint(self, path: str, tp_rank: int = 0, compress_config=None) -> None:
        """Writes this rank's slot-layout tensors under the serving key scheme (what
        `from_checkpoint` reads back without conversion)."""
        from safetensors.torch import save_file
        os.makedirs(path, exist_ok=True)
        tensors = {}
        for name, d in self.deltas.items():
            if d._compressed:
                tensors[f"{name}.{tp_rank}.qweight"] = d.qweight.clone().contiguous()
                tensors[f"{name}.{tp_rank}.scales"] = d.scales.clone().contiguous()
                tensors[f"{name}.{tp_rank}.meta"] = d.meta.clone().contiguous()
        save_file(tensors, os.path.join(path, "deltazip-compressed.safetensors"))
        cfg = compress_config or next(iter(self.deltas.values())).compress_config
        cfg.save_pretrained(path)


class DeltaModelManager:
    """Keeps registered deltas (pinned host arenas) and the GPU slots of every delta layer."""

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
        self.layout = SlotLayout()
        self.table_modules: Dict[str, torch.nn.Module] = {}   # embedding / logits layers (full tables)
        self._slot_has_base_table: Dict[Tuple[str, int], bool] = {}
        self.arena: Optional[torch.Tensor] = None
        self.uploads = 0                                   # host-to-device copies issued so far
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
        """Replaces every supported linear by its delta layer.  The layers' slot stacks are
        strided views of one device arena [slots, bytes per slot], so that everything one GPU
        slot holds is contiguous."""
        targets = []
        for name, module in list(self.model.named_modules()):
            leaf = name.split(".")[-1]
            if leaf not in self.supported_delta_modules:
                continue
            packed = self.packed_modules_mapping.get(leaf, [leaf])
            if isinstance(module, LogitsProcessor) and hasattr(self.model, "lm_head"):
                # the logits processor is sized after the output matrix it is used with
                new = from_layer_logits_processor(module, self.model.lm_head, self.delta_slots,
                                                  self.delta_config)
                self._install(name, new)
                self.table_modules[name] = new
                continue
            new = from_layer(module, self.delta_slots, self.delta_config, packed, allocate=False)
            if new is module:
                continue
            if isinstance(new, VocabParallelEmbeddingWithDelta):
                new.create_delta_weights(self.delta_slots, self.delta_config)
                self._install(name, new)
                self.table_modules[name] = new
                continue
            n, k = module.weight.shape
            self.layout.add(name, n, k, self.delta_config.max_bitwidth)
            targets.append((name, new, n, k))
        if not targets:
            return
        self.arena = torch.zeros((self.delta_slots, self.layout.total), dtype=torch.uint8,
                                 device=self.device)
        bits = self.delta_config.max_bitwidth
        for name, new, n, k in targets:
            qo, qb, mo, mb, so, sb = self.layout.regions[name]
            qs, ms, ss = ops.slot_shapes(n, k, bits)
            storage = (self.arena[:, qo:qo + qb].view(torch.int32).unflatten(1, qs),
                       self.arena[:, mo:mo + mb].view(torch.int16).unflatten(1, ms),
                       self.arena[:, so:so + sb].view(torch.float16).unflatten(1, ss))
            new.create_delta_weights(self.delta_slots, self.delta_config, storage=storage)
            self._install(name, new)
            self.modules[name] = new

    def _install(self, name: str, new: torch.nn.Module) -> None:
        parent = self.model
        parts = name.split(".")
        for p in parts[:-1]:
            parent = getattr(parent, p)
        setattr(parent, parts[-1], new)
        new.set_mapping(self.base_indices, self.sampler_indices, self.sampler_indices_padded,
                        self.embeddings_indices, self.indices_len, segments=self.segments)

    # -- registry ----------------------------------------------------------------
    def add_delta(self, delta: DeltaModel) -> bool:
        """Registers a delta in the host cache and packs it into its pinned arena."""
        if delta is None:
            raise ValueError("no delta to register (the load failed)")
        if delta.id in self._registered_deltas:
            return False
        if len(self._registered_deltas) >= self.capacity:
            raise RuntimeError("No free Delta slots.")
        self._check_and_pack(delta)
        self._registered_deltas[delta.id] = delta
        return True

    def _check_and_pack(self, delta: DeltaModel) -> None:
        for name, d in delta.deltas.items():
            if name not in self.modules or not d._compressed:
                continue
            if d.compress_config is not None and d.compress_config.bits != self.modules[name].bits:
                raise ValueError(f"{name}: {d.compress_config.bits}-bit delta in a "
                                 f"{self.modules[name].bits}-bit stack")
        if all((not d._compressed) or (not d.qweight.is_cuda) for d in delta.deltas.values()):
            delta.pack(self.layout)

    def remove_delta(self, delta_id: int) -> bool:
        self.deactivate_delta(delta_id)
        return bool(self._registered_deltas.pop(delta_id, None))

    def list_deltas(self) -> Dict[int, DeltaModel]:
        return dict(self._registered_deltas)

    def get_delta(self, delta_id: int) -> Optional[DeltaModel]:
        return self._registered_deltas.get(delta_id)

    # -- GPU slots ---------------------------------------------------------------
    def _upload(self, delta: DeltaModel, index: int) -> None:
        """Enqueues the upload of `delta` into slot `index` on the copy stream: one copy of the
        delta's pinned arena into the slot's device arena.  The copy only waits for the compute
        work that was enqueued before the slot was last released (an event), so it overlaps
        with whatever the compute stream is running now."""
        L = lib()
        cs = self.copy_stream.cuda_stream
        rel = self._slot_released[index]
        if rel is not None:
            self.copy_stream.wait_event(rel)
        for name, module in self.modules.items():
            module.bitwidth[index] = delta.bitwidth
        if delta.arena is not None and delta._arena_layout is self.layout:
            check(L.dz_slot_upload(self.arena[index].data_ptr(), delta.arena.data_ptr(),
                                   self.layout.total, 0, cs), "dz_slot_upload")
            self.uploads += 1
        else:
            # device-resident sources (tests, synthetic deltas): per-tensor device copies
            with torch.cuda.stream(self.copy_stream):
                for name, module in self.modules.items():
                    d = delta.get_delta(name)
                    if d is None or not d._compressed:
                        module.reset_delta(index)
                        continue
                    module.qweight_stacked[index].copy_(d.qweight.reshape(module.qweight_stacked[index].shape),
                                                        non_blocking=True)
                    module.scales_stacked[index].copy_(d.scales.reshape(module.scales_stacked[index].shape),
                                                       non_blocking=True)
                    module.meta_stacked[index].copy_(d.meta.reshape(module.meta_stacked[index].shape),
                                                     non_blocking=True)
                    self.uploads += 3
                ops.stream_fence()
        # replacement tables (embedding, output matrix) of deltas that carry them
        with torch.cuda.stream(self.copy_stream):
            for name, module in self.table_modules.items():
                d = delta.get_delta(name) or delta.get_delta(name.replace("logits_processor", "lm_head"))
                if d is not None and d.weight is not None:
                    module.set_delta(index, delta.bitwidth, d.weight)
                    self._slot_has_base_table[(name, index)] = False
                elif not self._slot_has_base_table.get((name, index), False):
                    # tables replace, they do not add: a delta without its own table serves
                    # the base model's (copied once; later table-less deltas reuse the copy)
                    base = self.model.lm_head.weight if isinstance(module, LogitsProcessorWithDelta) \
                        else module.base_layer.weight
                    module.set_delta(index, delta.bitwidth, base)
                    self._slot_has_base_table[(name, index)] = True
        ev = torch.cuda.Event()
        ev.record(self.copy_stream)
        self._slot_ready[index] = ev

    def _free_slot(self) -> Optional[int]:
        return next((i for i, d in enumerate(self.delta_index_to_id)
                     if d is None and i not in self._loading.values()), None)

    def prefetch_delta(self, delta_id: int) -> bool:
        """Starts moving a registered delta into a free GPU slot without making the compute
        stream wait (the reference prefetches only disk -> pinned host,
        serving/vllm/delta/worker_manager.py:324-333; here the host -> device leg overlaps with
        decode as well).  The slot is reserved; activate_delta later publishes it.  Returns
        False when the delta is already on the GPU or no slot is free."""
        if delta_id in self._active_deltas or delta_id in self._loading:
            return False
        index = self._free_slot()
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
            index = self._free_slot()
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

    def adopt_resident(self, delta_id: int, index: int) -> None:
        """Declares that slot `index` already holds delta `delta_id`: the caller wrote the slot
        tensors on the device itself (synthetic deltas generated in place)."""
        if self.delta_index_to_id[index] is not None or index in self._loading.values():
            raise ValueError(f"slot {index} is occupied")
        self.delta_index_to_id[index] = delta_id
        self._active_deltas[delta_id] = None
        for module in self.modules.values():
            module.bitwidth[index] = self.delta_config.max_bitwidth
        ops.stream_fence()        # the caller's slot writes never directly precede an SBMM
        self._last_mapping = None

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
        (base, sampler, padded, emb, indices_len), (is_sorted, runs) = _convert_mapping(
            mapping, self.delta_index_to_id, self.delta_slots + 1, self.vocab_size,
            self.delta_config.delta_extra_vocab_size, device=self.device)
        self.base_indices[: base.shape[0]].copy_(base)
        self.sampler_indices[: sampler.shape[0]].copy_(sampler)
        self.sampler_indices_padded[: padded.shape[0]].copy_(padded)
        self.embeddings_indices[: emb.shape[0], : emb.shape[1]].copy_(emb)
        self.indices_len[:] = indices_len
        # the host already knows the slot order: no device round trip for the sorted promise
        self.segments.build(self.base_indices[: base.shape[0]], sorted_hint=is_sorted)
        self.segments.host_runs = runs

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
        if delta is None:
            raise ValueError("no delta to register (the load failed)")
        if delta.id in self._registered_deltas:
            self._registered_deltas.move_to_end(delta.id)
            return False
        while len(self._registered_deltas) >= self.capacity:
            old, _ = next(iter(self._registered_deltas.items()))
            self.remove_delta(old)
        self._check_and_pack(delta)
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
        if delta_id in self._registered_deltas:
            self._registered_deltas.move_to_end(delta_id)
        return ok

    def remove_oldest_delta(self) -> bool:
        if not self._registered_deltas:
            return False
        old, _ = next(iter(self._registered_deltas.items()))
        return self.remove_delta(old)
