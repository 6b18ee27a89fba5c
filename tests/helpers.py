"""Shared helpers of the parity tests: seeded cases, numpy views, tolerance checks."""
from __future__ import annotations

import numpy as np
import torch

from yasakani_b200 import synth

ATOL, RTOL = 2e-3, 1e-2      # attention parity bar: max-abs 2e-3 / relative 1e-2 against the fp32-softmax oracle


def f16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_f16(a: np.ndarray) -> np.ndarray:
    return a.view(np.float16).astype(np.float32)


def build_oracle_cache(oracle, shape: synth.Shape, ctx: int, seed: int, max_ctx: int | None = None, chunk: int | None = None):
    """Oracle-side cache holding `ctx` appended tokens; returns (cache, k16, v16) with k16/v16 fp16 bit arrays."""
    max_ctx = max_ctx or ((ctx + 64 + 63) // 64) * 64
    k, v = synth.make_kv(shape, ctx, seed)
    k16, v16 = f16_bits(k), f16_bits(v)
    kv = oracle.KvCache(shape.hkv, shape.hd, max_ctx)
    step = chunk or ctx
    for p in range(0, ctx, step):
        oracle.append(kv, p, k16[p:p + step], v16[p:p + step])
    return kv, k16, v16


def assert_close(got: np.ndarray, want: np.ndarray, what: str, atol: float = ATOL, rtol: float = RTOL):
    got = np.asarray(got, np.float32); want = np.asarray(want, np.float32)
    err = np.abs(got - want)
    bad = err > (atol + rtol * np.abs(want))
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} outside atol {atol} rtol {rtol}; max abs err {err.max():.3e}"
    return float(err.max())
