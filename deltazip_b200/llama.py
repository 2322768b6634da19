"""A minimal Llama decoder over the delta linear layers: the harness that drives the SBMM
path the way the reference's model code does (serving/vllm/model_executor/models/llama.py
:59-235: qkv_proj -> rotary attention -> o_proj, gate_up_proj -> SiLU*up -> down_proj, RMSNorm,
module names and `supported_delta_modules` / `packed_modules_mapping` as in :299-327).

Only the four projections per layer are this library's work; attention, norms, rotary and the
sampler are plain PyTorch (they are not on the hot path).  Sequences advance in lock step with
a dense per-sequence KV cache, which is enough to check greedy decoding against the reference's
PyTorch dequantise-then-matmul path on random-init weights and to time decode steps.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import layers as L


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


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def rotary(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [B, T, H, D] (neox style, halves rotated), positions: [B, T]."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.float()[..., None] * inv                      # [B, T, D/2]
    cos, sin = ang.cos()[:, :, None, :], ang.sin()[:, :, None, :]
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, device="cuda"):
        super().__init__()
        kv = cfg.num_key_value_heads or cfg.num_attention_heads
        self.cfg = cfg
        self.qkv_proj = L.QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads,
                                            kv, device=device)
        self.o_proj = L.RowParallelLinear(cfg.hidden_size, cfg.hidden_size, device=device)
        self.gate_up_proj = L.MergedColumnParallelLinear(
            cfg.hidden_size, [cfg.intermediate_size, cfg.intermediate_size], device=device)
        self.down_proj = L.RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, device=device)
        self.input_layernorm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=torch.float16, device=device))
        self.post_attention_layernorm = nn.Parameter(
            torch.ones(cfg.hidden_size, dtype=torch.float16, device=device))


class LlamaForCausalLM(nn.Module):
    supported_delta_modules = ["qkv_proj", "o_proj", "gate_up_proj", "down_proj"]
    packed_modules_mapping = {"qkv_proj": ["q_proj", "k_proj", "v_proj"],
                              "gate_up_proj": ["gate_proj", "up_proj"]}

    def __init__(self, cfg: LlamaConfig, device="cuda", seed: int = 0):
        super().__init__()
        self.cfg = cfg
        g = torch.Generator(device=device).manual_seed(seed)
        self.embed_tokens = nn.Parameter(
            torch.empty((cfg.vocab_size, cfg.hidden_size), dtype=torch.float16, device=device).normal_(
                0, 1.0, generator=g), requires_grad=False)
        self.layers = nn.ModuleList([LlamaDecoderLayer(cfg, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=torch.float16, device=device))
        self.lm_head = nn.Parameter(
            torch.empty((cfg.vocab_size, cfg.hidden_size), dtype=torch.float16, device=device).normal_(
                0, 0.05, generator=g), requires_grad=False)
        # a custom linear hook lets the same model run the reference's PyTorch path
        self.linear_override: Optional[Callable[[str, nn.Module, torch.Tensor], torch.Tensor]] = None

    def _linear(self, name: str, module: nn.Module, x: torch.Tensor) -> torch.Tensor:
        if self.linear_override is not None:
            return self.linear_override(name, module, x)
        return module(x)[0]

    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, kv_cache: List[Dict],
                cache_len: int) -> torch.Tensor:
        """tokens, positions: [B, T]; kv_cache[layer] = {"k","v"}: [B, Hkv, Tmax, D]; returns the
        hidden states [B, T, hidden] after the final norm.  The B*T token rows are handed to the
        linear layers in (sequence, position) order."""
        cfg = self.cfg
        b, t = tokens.shape
        h = self.embed_tokens[tokens]                                  # [B, T, hidden]
        hkv = cfg.num_key_value_heads or cfg.num_attention_heads
        for li, layer in enumerate(self.layers):
            x = rms_norm(h, layer.input_layernorm, cfg.rms_norm_eps).reshape(b * t, -1)
            qkv = self._linear(f"layers.{li}.qkv_proj", layer.qkv_proj, x).reshape(b, t, -1)
            qd, kd = cfg.num_attention_heads * cfg.head_dim, hkv * cfg.head_dim
            q = rotary(qkv[..., :qd].reshape(b, t, cfg.num_attention_heads, cfg.head_dim), positions,
                       cfg.rope_theta)
            k = rotary(qkv[..., qd:qd + kd].reshape(b, t, hkv, cfg.head_dim), positions, cfg.rope_theta)
            v = qkv[..., qd + kd:].reshape(b, t, hkv, cfg.head_dim)
            kc, vc = kv_cache[li]["k"], kv_cache[li]["v"]
            kc[:, :, cache_len:cache_len + t] = k.transpose(1, 2)
            vc[:, :, cache_len:cache_len + t] = v.transpose(1, 2)
            keys, vals = kc[:, :, :cache_len + t], vc[:, :, :cache_len + t]
            if hkv != cfg.num_attention_heads:
                rep = cfg.num_attention_heads // hkv
                keys, vals = keys.repeat_interleave(rep, dim=1), vals.repeat_interleave(rep, dim=1)
            mask = None
            if t > 1:
                mask = torch.ones(t, cache_len + t, dtype=torch.bool, device=tokens.device).tril(cache_len)
            att = F.scaled_dot_product_attention(q.transpose(1, 2), keys, vals, attn_mask=mask)
            att = att.transpose(1, 2).reshape(b * t, -1)
            h = h + self._linear(f"layers.{li}.o_proj", layer.o_proj, att).reshape(b, t, -1)
            x = rms_norm(h, layer.post_attention_layernorm, cfg.rms_norm_eps).reshape(b * t, -1)
            gu = self._linear(f"layers.{li}.gate_up_proj", layer.gate_up_proj, x)
            half = gu.shape[-1] // 2
            act = F.silu(gu[:, :half]) * gu[:, half:]
            h = h + self._linear(f"layers.{li}.down_proj", layer.down_proj, act).reshape(b, t, -1)
        return rms_norm(h, self.norm, cfg.rms_norm_eps)

    def logits(self, hidden_last: torch.Tensor) -> torch.Tensor:
        """fp32 logits of the last position of every sequence (sampler math, not the hot path)."""
        return hidden_last.float() @ self.lm_head.float().t()

    def new_kv_cache(self, batch: int, max_len: int):
        hkv = self.cfg.num_key_value_heads or self.cfg.num_attention_heads
        dev = self.embed_tokens.device
        return [{"k": torch.zeros((batch, hkv, max_len, self.cfg.head_dim), dtype=torch.float16, device=dev),
                 "v": torch.zeros((batch, hkv, max_len, self.cfg.head_dim), dtype=torch.float16, device=dev)}
                for _ in self.layers]


@torch.inference_mode()
def greedy_generate(model: LlamaForCausalLM, prompts: torch.Tensor, steps: int,
                    set_mapping: Callable[[int], None]) -> torch.Tensor:
    """Prefill `prompts` [B, T] then `steps` greedy decode steps; `set_mapping(tokens_per_seq)`
    installs the per-token delta mapping for a forward pass with that many tokens per sequence.
    Returns the generated ids [B, steps]."""
    b, t = prompts.shape
    kv = model.new_kv_cache(b, t + steps)
    pos = torch.arange(t, device=prompts.device)[None, :].expand(b, t)
    set_mapping(t)
    h = model(prompts, pos, kv, 0)
    nxt = model.logits(h[:, -1]).argmax(-1)
    out = [nxt]
    set_mapping(1)
    for s in range(1, steps):
        pos = torch.full((b, 1), t + s - 1, device=prompts.device, dtype=torch.long)
        h = model(nxt[:, None], pos, kv, t + s - 1)
        nxt = model.logits(h[:, -1]).argmax(-1)
        out.append(nxt)
    return torch.stack(out, dim=1)
