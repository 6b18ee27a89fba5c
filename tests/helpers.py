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


# ---- GPU side (only used by -m gpu tests) ----

def gpu_append_all(kv4, layer, k: torch.Tensor, v: torch.Tensor, passes, pos0: int = 0):
    """Append host rows k, v [n][hkv][hd] to a device KvLayer in passes of the given sizes."""
    dk, dv = k.cuda(), v.cuda()
    d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = 0
    for n in passes:
        d_pos.fill_(pos0 + p)
        kv4.launch_kv_append(layer, dk[p:p + n].contiguous(), dv[p:p + n].contiguous(), d_pos, int(n))
        p += int(n)
    torch.cuda.synchronize()
    return p


def gpu_attention(kv4, layer, q: torch.Tensor, pos0: int, splits: int, rope, shape, bv=None, gate=None):
    """attention + combine through the C ABI; returns o16 as float32 numpy [M][hq][hd] and the raw partials."""
    M = q.shape[0]
    dq = q.cuda().contiguous()
    d_pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
    pm.fill_(float("nan")); pl.fill_(float("nan")); pacc.fill_(float("nan"))      # every slot must be written
    kv4.launch_attention_gqa(dq, layer, M, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=q.dtype, device="cuda")
    kv4.launch_attn_combine_gqa(pm, pl, pacc, splits, M, o16, shape.hq, shape.g, bv=bv, gate=gate)
    torch.cuda.synchronize()
    return o16.float().cpu().numpy(), (pm.cpu().numpy(), pl.cpu().numpy(), pacc.cpu().numpy())


# ---------------------------------------------------------------- inputs of the attention block's row epilogue (kvx attn_post)
def _oracle():
    from oracle import kv4_oracle
    return kv4_oracle


def bf16_bits(x: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).bfloat16().view(torch.int16).numpy().view(np.uint16).copy()


def post_inputs(seed, M, nh, kvh, rd, max_ctx, theta=1e7):
    """Seeded projection rows (bf16 bits), norm weights, rope table.  Returns a dict of numpy arrays."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((M, nh, 512)) * np.exp(rng.uniform(-1.0, 1.5, (1, nh, 1)))
    k = rng.standard_normal((M, kvh, 256)) * np.exp(rng.uniform(np.log(0.5), np.log(4.0), (1, kvh, 256)))
    v = rng.standard_normal((M, kvh, 256))
    if M > 1:
        q[1, 0, :256] = 0.0                      # an all-zero query head: r = 1 / sqrt(eps)
        k[1, 0] = 0.0                            # an all-zero key row: scale 0, payload 0
        v[1, kvh - 1] = 0.0
        k[0, kvh - 1] *= 3e3                     # large values
    rope = _oracle().rope_table(max_ctx, theta, rd) if rd else np.zeros((max_ctx, 0, 2), dtype=np.float32)
    return dict(q_rows=bf16_bits(q), k_rows=bf16_bits(k), v_rows=bf16_bits(v),
                qn_w=bf16_bits(rng.standard_normal(256) * 0.2), kn_w=bf16_bits(rng.standard_normal(256) * 0.2 + 0.5),
                rope=np.ascontiguousarray(rope, dtype=np.float32))
