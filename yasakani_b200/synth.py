"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

Q, K, V ~ N(0,1) rounded to bf16; K multiplied per (kv-head, channel) by exp(U(ln 0.5, ln 4)) (outlier
channels) and rounded to bf16 again; then converted to fp16 (the dtype the Family-A operators take).
seed = 1234 + 100 * config_index + sequence_index.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Shape:
    hq: int
    hkv: int
    hd: int
    rd: int
    theta: float

    @property
    def g(self) -> int:
        return self.hq // self.hkv

    @property
    def qscale(self) -> float:
        return 1.0 / math.sqrt(self.hd)

    def decode_bytes(self, ctx: int) -> int:
        """Algorithmic bytes of one decode step over `ctx` cached tokens: packed K and V rows, per-token V
        scale/zero, per-group K scale/zero, plus Q in and O out (16-bit)."""
        groups = (ctx + 31) // 32
        return self.hkv * (ctx * (self.hd // 2 + self.hd // 2 + 4) + groups * self.hd * 4) + 2 * self.hq * self.hd * 2

    def attn_flops(self, keys_total: int) -> int:
        """4 * HD * Hq * (sum over rows of visible keys): QK^T and PV, multiply and add."""
        return 4 * self.hd * self.hq * keys_total


C1 = Shape(hq=16, hkv=2, hd=128, rd=128, theta=1e6)     # CPU-runnable reference case
C2 = Shape(hq=24, hkv=4, hd=256, rd=64, theta=1e7)      # 27B-class full-attention layer


def seed_for(config_index: int, sequence_index: int = 0) -> int:
    return 1234 + 100 * config_index + sequence_index


def make_kv(shape: Shape, n_tokens: int, seed: int, dtype=torch.float16):
    """K, V rows [n_tokens][Hkv][HD] (host tensors)."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn((n_tokens, shape.hkv, shape.hd), generator=g, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn((n_tokens, shape.hkv, shape.hd), generator=g, dtype=torch.float32).to(torch.bfloat16)
    lo, hi = math.log(0.5), math.log(4.0)
    ch = torch.exp(torch.rand((shape.hkv, shape.hd), generator=g, dtype=torch.float32) * (hi - lo) + lo)
    k = (k.float() * ch).to(torch.bfloat16)
    return k.to(dtype), v.to(dtype)


def make_q(shape: Shape, rows: int, seed: int, dtype=torch.float16):
    """Q rows [rows][Hq][HD] (host tensor), a stream independent of make_kv's."""
    g = torch.Generator().manual_seed(seed + 7919)
    return torch.randn((rows, shape.hq, shape.hd), generator=g, dtype=torch.float32).to(torch.bfloat16).to(dtype)
