"""Configuration objects of the delta plugin, field for field those of the reference
(serving/vllm/delta/config.py:20-104) minus its back-end switches (one kernel here)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from fractions import Fraction
from os.path import join
from typing import Optional

import torch


@dataclass
class CompressionConfig:
    """How a delta was compressed (compress_config.json next to the checkpoint)."""
    bits: int = 4
    sparsity: float = 0.0
    prunen: int = 0
    prunem: int = 0
    group_size: int = -1
    group_rows: int = -1
    block_size: int = 128
    damp_percent: float = 0.01
    desc_act: bool = True
    sym: bool = True
    true_sequential: bool = True
    lossless: str = "none"
    dtype: str = "fp16"
    pack_factor: Fraction = field(default=Fraction(32, 1))

    def __post_init__(self):
        if not 0 <= self.sparsity <= 1:
            raise ValueError(f"sparsity {self.sparsity} lies outside [0, 1]")
        if self.bits not in (2, 3, 4, 8, 16):
            raise ValueError(f"{self.bits}-bit codes are not a supported width (2, 3, 4, 8, 16)")
        if self.group_size != -1 and self.group_size <= 0:
            raise ValueError("group_size is -1 (one group per row) or a positive count")
        if not 0 < self.damp_percent < 1:
            raise ValueError(f"damp_percent {self.damp_percent} lies outside (0, 1)")
        self.pack_factor = Fraction(32, self.bits)

    def to_dict(self):
        return {k: getattr(self, k) for k in (
            "bits", "group_size", "sparsity", "damp_percent", "desc_act", "sym", "true_sequential",
            "lossless", "prunen", "prunem", "block_size")}

    def save_pretrained(self, save_dir: str):
        with open(join(save_dir, "compress_config.json"), "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2)

    @classmethod
    def from_pretrained(cls, save_dir: str) -> "CompressionConfig":
        with open(join(save_dir, "compress_config.json"), "r", encoding="utf-8") as f:
            return cls(**json.load(f))

    def servable(self) -> bool:
        """True when the SBMM kernel can serve this delta: 2:4 sparse, symmetric, 2 or 4 bit,
        one scale per output channel."""
        return (self.bits in (2, 4) and self.sym and self.group_size == -1
                and self.prunen == 2 and self.prunem == 4)


@dataclass
class DeltaConfig:
    """Serving-side limits: GPU slots, pinned-CPU cache size, widest bit width."""
    max_deltas: int = 1
    max_bitwidth: int = 4
    delta_dtype: Optional[torch.dtype] = torch.int32
    max_cpu_deltas: Optional[int] = None
    delta_extra_vocab_size: int = 0
    pack_factor: Fraction = field(default=Fraction(32, 1))
    sparse_factor: Fraction = field(default=Fraction(2, 1))

    def __post_init__(self):
        if self.max_cpu_deltas is None:
            self.max_cpu_deltas = self.max_deltas
        elif self.max_cpu_deltas < self.max_deltas:
            raise ValueError("the pinned-host cache (max_cpu_deltas) cannot be smaller than the GPU slots (max_deltas)")
        if self.max_bitwidth not in (2, 4):
            raise ValueError("max_bitwidth must be 2 or 4")
        self.pack_factor = Fraction(32, self.max_bitwidth)
