"""A small decode engine over the delta layers: sequences, the paged KV cache, delta-aware
admission and the per-step device state.  It stands where the reference's scheduler and model
runner stand around the SBMM path (serving/vllm/core/scheduler.py:359-366,528-535: a batch may
hold at most `max_deltas` distinct deltas and is sorted by delta id, :101-104;
serving/vllm/worker/model_runner.py:919-975: set the active deltas and the mapping, run the
model, sample) -- reduced to greedy sampling and to what the throughput configurations need.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .config import DeltaConfig
from .layers import DeltaMapping
from .llama import AttnMeta, LlamaConfig, LlamaForCausalLM, PagedKVCache
from .models import LRUCacheDeltaModelManager


@dataclass
class Sequence:
    seq_id: int
    delta_id: int                       # 0 = base model
    length: int                         # tokens in the cache so far
    max_new: int
    blocks: List[int] = field(default_factory=list)
    generated: int = 0
    arrival: float = 0.0
    prompt: Optional[torch.Tensor] = None
    first_token_time: Optional[float] = None


class DecodeEngine:
    """Model + slot manager + KV cache for one tensor-parallel rank."""

    def __init__(self, cfg: LlamaConfig, delta_config: DeltaConfig, max_seqs: int, kv_blocks: int,
                 block_size: int = 16, device="cuda", dtype=torch.float16, seed: int = 0):
        self.cfg, self.device, self.block_size = cfg, torch.device(device), block_size
        self.model = LlamaForCausalLM(cfg, device=device, seed=seed, dtype=dtype)
        self.manager = LRUCacheDeltaModelManager(self.model, max_seqs, max(max_seqs, 2048),
                                                 cfg.vocab_size, delta_config, device=device)
        self.cache = PagedKVCache(cfg.num_hidden_layers, kv_blocks, self.model.kv_heads, block_size,
                                  dtype, device)
        self.max_seqs = max_seqs
        self.running: List[Sequence] = []
        self._dirty = True
        self._order: List[int] = []
        self.tokens = None
        self.positions = None
        self.block_tables = None
        self.attn_splits = 0            # 0: chosen per step from the batch (see decode_step)
        self.swap_ins = 0

    # -- batch composition -----------------------------------------------------------
    def admit(self, waiting: List[Sequence]) -> List[Sequence]:
        """Delta-aware admission: sequences join while a batch slot, KV blocks for their whole
        life and a GPU slot for their delta are available.  A delta that is not resident takes a
        free slot or evicts the least recently used delta no running sequence needs.  Returns
        the sequences admitted (their deltas are resident and activated)."""
        admitted = []
        mgr = self.manager
        in_use = {s.delta_id for s in self.running if s.delta_id > 0}
        for seq in list(waiting):
            if len(self.running) + len(admitted) >= self.max_seqs:
                break
            need = (seq.length + seq.max_new + self.block_size - 1) // self.block_size
            if need > len(self.cache.free):
                continue
            d = seq.delta_id
            if d > 0 and d not in mgr._active_deltas:
                if mgr.get_delta(d) is None:
                    continue                                    # unknown delta: not servable
                if len(mgr._active_deltas) + len(mgr._loading) >= mgr.delta_slots and d not in mgr._loading:
                    victim = next((x for x in mgr._active_deltas if x not in in_use), None)
                    if victim is None:
                        continue                                # every slot is needed by the batch
                    mgr.deactivate_delta(victim)
                mgr.activate_delta(d)
            elif d > 0:
                mgr._active_deltas.move_to_end(d)
            in_use.add(d)
            seq.blocks = self.cache.allocate(need)
            admitted.append(seq)
            waiting.remove(seq)
        if admitted:
            self.running.extend(admitted)
            self._dirty = True
        return admitted

    def admit_overlapped(self, waiting: List[Sequence], ready=None) -> List[Sequence]:
        """Admission that never makes the compute stream wait for a swap-in: a sequence whose
        delta is not resident triggers a prefetch into a free (or evictable) GPU slot -- the
        upload runs on the copy stream while the batch keeps decoding -- and joins in a later
        round, once the upload's event has completed.  `ready(delta_id) -> bool` reports that
        (default: the event's own query; a tensor-parallel caller passes the agreement of all
        ranks so that every rank admits the same sequences)."""
        mgr = self.manager
        if ready is None:
            def ready(d):
                return mgr._slot_ready[mgr._loading[d]].query()
        admitted = []
        in_use = {s.delta_id for s in self.running if s.delta_id > 0}
        wanted = set()
        for seq in list(waiting):
            if len(self.running) + len(admitted) >= self.max_seqs:
                break
            need = (seq.length + seq.max_new + self.block_size - 1) // self.block_size
            if need > len(self.cache.free):
                continue
            d = seq.delta_id
            if d > 0 and d not in mgr._active_deltas:
                if mgr.get_delta(d) is None:
                    continue
                if d in mgr._loading:
                    if not ready(d):
                        continue
                    mgr.activate_delta(d)              # upload finished: no stall
                else:
                    if d in wanted:
                        continue
                    if len(mgr._active_deltas) + len(mgr._loading) >= mgr.delta_slots:
                        victim = next((x for x in mgr._active_deltas if x not in in_use), None)
                        if victim is None:
                            continue
                        mgr.deactivate_delta(victim)
                    mgr.prefetch_delta(d)
                    self.swap_ins += 1
                    wanted.add(d)
                    continue
            elif d > 0:
                mgr._active_deltas.move_to_end(d)
            in_use.add(d)
            seq.blocks = self.cache.allocate(need)
            admitted.append(seq)
            waiting.remove(seq)
        if admitted:
            self.running.extend(admitted)
            self._dirty = True
        return admitted

    def retire(self, seq: Sequence) -> None:
        self.cache.release(seq.blocks)
        seq.blocks = []
        self.running.remove(seq)
        self._dirty = True

    def _slot_of(self, delta_id: int) -> int:
        return self.manager.delta_index_to_id.index(delta_id) if delta_id > 0 else -1

    def _rebuild(self, tokens: Optional[Dict[int, int]] = None) -> None:
        """Device-side state of the running batch, sequences ordered by GPU slot so that the
        token rows reach the SBMM sorted.  `tokens`: seq_id -> next input token."""
        old = {}
        if self.tokens is not None and self._order:
            host = self.tokens.tolist()
            old = {sid: host[i] for i, sid in enumerate(self._order)}
        if tokens:
            old.update(tokens)
        self.running.sort(key=lambda s: (self._slot_of(s.delta_id), s.seq_id))
        self._order = [s.seq_id for s in self.running]
        dev = self.device
        b = len(self.running)
        maxb = max((len(s.blocks) for s in self.running), default=1)
        tab = torch.zeros((max(b, 1), maxb), dtype=torch.int32)
        for i, s in enumerate(self.running):
            tab[i, : len(s.blocks)] = torch.tensor(s.blocks, dtype=torch.int32)
        self.block_tables = tab.to(dev)
        self.positions = torch.tensor([s.length for s in self.running], dtype=torch.int64, device=dev)
        self.tokens = torch.tensor([old.get(s.seq_id, 0) for s in self.running], dtype=torch.int64,
                                   device=dev)
        ids = [s.delta_id for s in self.running]
        self.manager.set_delta_mapping(DeltaMapping(ids, ids))
        self._dirty = False

    # -- one decode step ---------------------------------------------------------------
    @torch.inference_mode()
    def decode_step(self) -> torch.Tensor:
        """Feeds every running sequence its latest token (position = its cached length), appends
        the new key/value to the cache and samples the next token greedily.  Device work only
        unless the batch composition changed since the last step."""
        if self._dirty:
            self._rebuild()
        bs = self.block_size
        pos = self.positions
        blk = torch.gather(self.block_tables, 1, (pos // bs).unsqueeze(1)).squeeze(1).to(torch.int64)
        slot = blk * bs + pos % bs
        lens = (pos + 1).to(torch.int32)
        # one CTA per (sequence, kv head, split): split the keys when the batch alone would leave
        # most SMs without a CTA
        splits = self.attn_splits or max(1, min(8, 296 // max(1, len(self.running) * self.model.kv_heads)))
        h = self.model(self.tokens, pos, self.cache,
                       AttnMeta(slot_mapping=slot, block_tables=self.block_tables, seq_lens=lens,
                                splits=splits))
        self.tokens = self.model.greedy_tokens(h)
        self.positions = pos + 1
        for s in self.running:
            s.length += 1
            s.generated += 1
        return self.tokens

    @torch.inference_mode()
    def prefill(self, seqs: List[Sequence]) -> None:
        """Runs the prompts of newly admitted sequences (all tokens of all prompts in one pass,
        rows sorted by GPU slot), fills their cache blocks and leaves their first generated token
        as the next decode input."""
        if not seqs:
            return
        seqs = sorted(seqs, key=lambda s: (self._slot_of(s.delta_id), s.seq_id))
        dev = self.device
        toks = torch.cat([s.prompt for s in seqs]).to(dev)
        pos = torch.cat([torch.arange(s.prompt.numel()) for s in seqs]).to(dev)
        slots = torch.tensor([x for s in seqs for x in self.cache.slots(s.blocks, 0, s.prompt.numel())],
                             dtype=torch.int64, device=dev)
        lens = [int(s.prompt.numel()) for s in seqs]
        ids = [s.delta_id for s in seqs for _ in range(int(s.prompt.numel()))]
        self.manager.set_delta_mapping(DeltaMapping(ids, [s.delta_id for s in seqs]))
        h = self.model(toks, pos, self.cache, AttnMeta(slot_mapping=slots, prompt_lens=lens))
        last = torch.tensor(lens, device=dev).cumsum(0) - 1
        nxt = self.model.greedy_tokens(h[last]).tolist()
        first = {s.seq_id: nxt[i] for i, s in enumerate(seqs)}
        for s in seqs:
            s.length = int(s.prompt.numel())
            s.generated = 1
        self._rebuild(first)
