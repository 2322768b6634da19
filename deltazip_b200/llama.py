"""A minimal Llama decoder over the delta linear layers: the harness that drives the SBMM
path the way the reference's model code does (serving/vllm/model_executor/models/llama.py
:59-235: qkv_proj -> rotary attention -> o_proj, gate_up_proj -> SiLU*up -> down_proj, RMSNorm
with the residual carried beside the hidden state, module names and `supported_delta_modules` /
`packed_modules_mapping` as in :299-327), tensor parallel over the ranks of parallel_state.

A decode step is a chain of this library's launches: per layer rmsnorm (+ residual add), qkv
SBMM, rotary + paged-cache write, paged decode attention, o SBMM (+ all-reduce), rmsnorm, gate_up
SBMM, SiLU*up, down SBMM (+ all-reduce).  Prefill runs the same linears over all prompt tokens
and uses PyTorch's attention on the fresh q/k/v (prefill attention is not on the path).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import layers as L
from . import ops
from .parallel_state import (SHARD_UNIT, get_tensor_model_parallel_rank,
                             get_tensor_model_parallel_world_size, shard_range)


@dataclass
class LlamaConfig:
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    vocab_size: int = 32000
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def kv_heads(self) -> int:
        return self.num_key_value_heads or self.num_attention_heads


LLAMA2_7B = LlamaConfig(4096, 11008, 32, 32, None)
LLAMA2_13B = LlamaConfig(5120, 13824, 40, 40, None)
LLAMA2_70B = LlamaConfig(8192, 28672, 80, 64, 8)


class PagedKVCache:
    """Per-layer K and V pools of `num_blocks` blocks of `block_size` tokens, [slots, kv_heads,
    128] each, with a free list (role of the reference's block manager + cache engine,
    serving/vllm/core/block_manager.py, serving/vllm/worker/cache_engine.py, reduced to what a
    single process needs)."""

    def __init__(self, num_layers: int, num_blocks: int, kv_heads: int, block_size: int = 16,
                 dtype=torch.float16, device="cuda"):
        self.block_size, self.num_blocks, self.kv_heads = block_size, num_blocks, kv_heads
        shape = (num_blocks * block_size, kv_heads, 128)
        self.k = [torch.empty(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.v = [torch.empty(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))

    def allocate(self, n_blocks: int) -> List[int]:
        if n_blocks > len(self.free):
            raise RuntimeError("out of KV cache blocks")
        return [self.free.pop() for _ in range(n_blocks)]

    def release(self, blocks: Sequence[int]) -> None:
        self.free.extend(blocks)

    def slots(self, blocks: Sequence[int], start: int, count: int) -> List[int]:
        """Cache slots of token positions [start, start + count) of a sequence owning `blocks`."""
        bs = self.block_size
        return [blocks[p // bs] * bs + p % bs for p in range(start, start + count)]


@dataclass
class AttnMeta:
    """How attention runs in one forward pass.  Decode: `block_tables` [B, max_blocks] int32 and
    `seq_lens` [B] int32 (cached length including the current token).  Prefill: `prompt_lens`,
    the token count of each sequence, rows in (sequence, position) order."""
    slot_mapping: Optional[torch.Tensor] = None          # int64 [M] cache slot per token, -1 = none
    block_tables: Optional[torch.Tensor] = None
    seq_lens: Optional[torch.Tensor] = None
    prompt_lens: Optional[List[int]] = None
    splits: int = 1


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, device="cuda", dtype=torch.float16):
        super().__init__()
        self.cfg = cfg
        self.qkv_proj = L.QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads,
                                            cfg.kv_heads, device=device, dtype=dtype)
        self.o_proj = L.RowParallelLinear(cfg.hidden_size, cfg.hidden_size, device=device, dtype=dtype)
        self.gate_up_proj = L.MergedColumnParallelLinear(
            cfg.hidden_size, [cfg.intermediate_size, cfg.intermediate_size], device=device, dtype=dtype)
        self.down_proj = L.RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, device=device,
                                             dtype=dtype)
        self.input_layernorm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device),
                                            requires_grad=False)
        self.post_attention_layernorm = nn.Parameter(
            torch.ones(cfg.hidden_size, dtype=dtype, device=device), requires_grad=False)


class LlamaForCausalLM(nn.Module):
    supported_delta_modules = ["qkv_proj", "o_proj", "gate_up_proj", "down_proj"]
    packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "v_proj"],
                              "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self, cfg: LlamaConfig, device="cuda", seed: int = 0, dtype=torch.float16):
        super().__init__()
        self.cfg = cfg
        self.dtype = dtype
        self.tp_size = get_tensor_model_parallel_world_size()
        self.tp_rank = get_tensor_model_parallel_rank()
        if cfg.head_dim != 128:
            raise ValueError("the decode kernels take head size 128 (every Llama-2 size)")
        if cfg.num_attention_heads % self.tp_size:
            raise ValueError("attention heads must divide by the tensor-parallel size")
        self.q_heads = cfg.num_attention_heads // self.tp_size
        self.kv_heads = max(1, cfg.kv_heads // self.tp_size)
        g = torch.Generator(device=device).manual_seed(seed)
        self.embed_tokens = nn.Parameter(
            torch.empty((cfg.vocab_size, cfg.hidden_size), dtype=dtype, device=device).normal_(
                0, 1.0, generator=g), requires_grad=False)
        self.layers = nn.ModuleList([LlamaDecoderLayer(cfg, device, dtype)
                                     for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device),
                                 requires_grad=False)
        # vocab-parallel output matrix: this rank's rows [v_lo, v_hi)
        full = torch.empty((cfg.vocab_size, cfg.hidden_size), dtype=dtype, device=device).normal_(
            0, 0.05, generator=g)
        self.v_lo, self.v_hi = shard_range(cfg.vocab_size, SHARD_UNIT, self.tp_rank, self.tp_size) \
            if cfg.vocab_size % SHARD_UNIT == 0 else (0, cfg.vocab_size)
        self.lm_head = nn.Parameter(full[self.v_lo:self.v_hi].contiguous(), requires_grad=False)
        del full
        # a custom linear hook lets the same model run the reference's PyTorch path
        self.linear_override: Optional[Callable[[str, nn.Module, torch.Tensor], torch.Tensor]] = None

    def _linear(self, name: str, module: nn.Module, x: torch.Tensor) -> torch.Tensor:
        if self.linear_override is not None:
            return self.linear_override(name, module, x)
        return module(x)[0]

    # -- attention ---------------------------------------------------------------
    def _attention(self, li: int, qkv: torch.Tensor, positions: torch.Tensor,
                   cache: Optional[PagedKVCache], meta: AttnMeta) -> torch.Tensor:
        cfg = self.cfg
        kc = cache.k[li] if cache is not None else None
        vc = cache.v[li] if cache is not None else None
        ops.rotary_and_cache(qkv, positions, self.q_heads, self.kv_heads, cfg.rope_theta, kc, vc,
                             meta.slot_mapping if cache is not None else None)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        if meta.prompt_lens is None:
            return ops.paged_attention_decode(qkv, kc, vc, meta.block_tables, meta.seq_lens,
                                              self.q_heads, self.kv_heads, cache.block_size, scale,
                                              splits=meta.splits)
        # prefill: causal attention of every prompt over its own fresh keys / values
        qd, kd = self.q_heads * 128, self.kv_heads * 128
        out = torch.empty((qkv.shape[0], qd), dtype=qkv.dtype, device=qkv.device)
        row = 0
        for t in meta.prompt_lens:
            blk = qkv[row:row + t]
            q = blk[:, :qd].reshape(t, self.q_heads, 128).transpose(0, 1)[None]
            k = blk[:, qd:qd + kd].reshape(t, self.kv_heads, 128).transpose(0, 1)[None]
            v = blk[:, qd + kd:].reshape(t, self.kv_heads, 128).transpose(0, 1)[None]
            if self.kv_heads != self.q_heads:
                rep = self.q_heads // self.kv_heads
                k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
            att = F.scaled_dot_product_attention(q, k, v, is_causal=t > 1, scale=scale)
            out[row:row + t] = att[0].transpose(0, 1).reshape(t, qd)
            row += t
        return out

    # -- forward -------------------------------------------------------------------
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, cache: Optional[PagedKVCache],
                meta: AttnMeta) -> torch.Tensor:
        """tokens, positions: [M] (int64); returns the hidden states [M, hidden] after the final
        norm.  Token rows are handed to the linear layers in the order given."""
        cfg = self.cfg
        eps = cfg.rms_norm_eps
        residual = self.embed_tokens[tokens]                            # [M, hidden]
        x = ops.rms_norm(residual, self.layers[0].input_layernorm, eps)
        for li, layer in enumerate(self.layers):
            if li > 0:
                x = ops.rms_norm(x, layer.input_layernorm, eps, residual=residual)
            qkv = self._linear(f"layers.{li}.qkv_proj", layer.qkv_proj, x)
            att = self._attention(li, qkv, positions, cache, meta)
            assert att.shape[-1] == layer.o_proj.weight.shape[1], "qkv shard does not feed o_proj's K"
            o = self._linear(f"layers.{li}.o_proj", layer.o_proj, att)
            x = ops.rms_norm(o, layer.post_attention_layernorm, eps, residual=residual)
            gu = self._linear(f"layers.{li}.gate_up_proj", layer.gate_up_proj, x)
            act = ops.silu_and_mul(gu)
            assert act.shape[-1] == layer.down_proj.weight.shape[1], \
                "gate/up shard does not feed down_proj's K"
            x = self._linear(f"layers.{li}.down_proj", layer.down_proj, act)
        return ops.rms_norm(x, self.norm, eps, residual=residual)

    # -- sampling --------------------------------------------------------------------
    def logits(self, hidden_last: torch.Tensor) -> torch.Tensor:
        """fp32 logits over this rank's vocabulary rows (sampler math, not the hot path)."""
        return hidden_last.float() @ self.lm_head.float().t()

    def greedy_tokens(self, hidden_last: torch.Tensor) -> torch.Tensor:
        """argmax over the whole vocabulary: the output matrix runs on the dense tcgen05 GEMM,
        each rank reduces its own vocabulary rows and the (value, index) pairs are exchanged
        (the reference gathers full logits to rank 0 instead,
        serving/vllm/delta/layers_marlin.py:696-711)."""
        logits = ops.base_gemm(hidden_last, self.lm_head) if self.lm_head.shape[0] % 128 == 0 \
            else (hidden_last @ self.lm_head.t())
        val, idx = logits.float().max(dim=-1)
        idx = idx + self.v_lo
        if self.tp_size == 1:
            return idx
        import torch.distributed as dist
        pair = torch.stack([val, idx.float()], dim=-1).contiguous()
        parts = [torch.empty_like(pair) for _ in range(self.tp_size)]
        dist.all_gather(parts, pair)
        allp = torch.stack(parts)                                       # [tp, B, 2]
        best = allp[:, :, 0].argmax(dim=0)
        return allp[best, torch.arange(pair.shape[0], device=pair.device), 1].long()


@torch.inference_mode()
def greedy_generate(model: LlamaForCausalLM, prompts: torch.Tensor, steps: int,
                    set_mapping: Callable[[int], None], block_size: int = 16) -> torch.Tensor:
    """Prefill `prompts` [B, T] then `steps` greedy decode steps; `set_mapping(tokens_per_seq)`
    installs the per-token delta mapping for a forward pass with that many tokens per sequence
    (rows in sequence-major order).  Returns the generated ids [B, steps]."""
    b, t = prompts.shape
    dev = prompts.device
    blocks_per_seq = (t + steps + block_size - 1) // block_size
    cache = PagedKVCache(len(model.layers), b * blocks_per_seq, model.kv_heads, block_size,
                         model.dtype, dev)
    tables = [cache.allocate(blocks_per_seq) for _ in range(b)]
    block_tables = torch.tensor(tables, dtype=torch.int32, device=dev)
    slots = torch.tensor([cache.slots(tb, 0, t) for tb in tables], dtype=torch.int64, device=dev)
    pos = torch.arange(t, device=dev)[None, :].expand(b, t)
    set_mapping(t)
    h = model(prompts.reshape(-1), pos.reshape(-1).contiguous(), cache,
              AttnMeta(slot_mapping=slots.reshape(-1), prompt_lens=[t] * b))
    nxt = model.logits(h.reshape(b, t, -1)[:, -1]).argmax(-1)
    out = [nxt]
    set_mapping(1)
    for s in range(1, steps):
        cur = t + s - 1                                                  # position of the token fed in
        pos1 = torch.full((b,), cur, device=dev, dtype=torch.int64)
        slot1 = torch.tensor([cache.slots(tb, cur, 1)[0] for tb in tables], dtype=torch.int64, device=dev)
        lens = torch.full((b,), cur + 1, device=dev, dtype=torch.int32)
        h = model(nxt, pos1, cache, AttnMeta(slot_mapping=slot1, block_tables=block_tables, seq_lens=lens))
        nxt = model.logits(h).argmax(-1)
        out.append(nxt)
    return torch.stack(out, dim=1)
