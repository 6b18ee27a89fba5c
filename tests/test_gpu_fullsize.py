"""Benchmark-sized cases (BASELINE.json configs 2, 3 and 5) on the GPU: sampled rows against the CPU oracle, plus
properties that need no oracle (bitwise width invariance, tensor-core kernel against the CUDA-core kernel)."""
import numpy as np
import pytest
import torch

from tests.helpers import assert_close, f16_bits
from yasakani_b200 import synth, ALGO_AUTO, ALGO_SCALAR

pytestmark = pytest.mark.gpu
CHUNK = 8192


def _build(kv4, oracle, shape, n_tokens, seed, want_oracle=True):
    """GPU cache (library codec) and, optionally, the oracle's cache from the same seeded rows, chunk by chunk."""
    max_ctx = ((n_tokens + 127) // 64) * 64
    layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
    okv = oracle.KvCache(shape.hkv, shape.hd, max_ctx) if want_oracle else None
    d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    for c in range((n_tokens + CHUNK - 1) // CHUNK):
        n = min(CHUNK, n_tokens - c * CHUNK)
        k, v = synth.make_kv(shape, CHUNK, seed=seed * 1000 + c)
        d_pos.fill_(c * CHUNK)
        kv4.launch_kv_append(layer, k[:n].cuda(), v[:n].cuda(), d_pos, n)
        if want_oracle:
            oracle.append(okv, c * CHUNK, f16_bits(k[:n]), f16_bits(v[:n]))
    torch.cuda.synchronize()
    return layer, okv, max_ctx


def _rope(kv4, shape, max_ctx):
    rope = torch.empty((max_ctx, shape.rd // 2, 2), dtype=torch.float32, device="cuda")
    kv4.launch_rope_table_g(rope, max_ctx, shape.theta, shape.rd)
    torch.cuda.synchronize()
    return rope


def test_config5_prefill_8192_rows_sampled_against_oracle(oracle):
    from yasakani_b200 import kv4
    shape, M = synth.C2, 8192
    layer, okv, max_ctx = _build(kv4, oracle, shape, M, seed=71)
    got_cache = layer.to_numpy()
    for name, want in okv.arrays().items():                              # the prompt's K/V went through the codec: bit-exact
        assert np.array_equal(got_cache[name].reshape(want.shape), want), name
    rope = _rope(kv4, shape, max_ctx)
    q = synth.make_q(shape, M, seed=71)
    d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, 1, shape.hq, shape.hd)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_attention_prefill_tc(q.cuda(), layer, M, d_pos, 1, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, kv4.tc_workspace(layer, M))
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
    got = o16.float().cpu().numpy()
    assert np.isfinite(got).all()
    rope_np = rope.cpu().numpy()
    for lo, hi in ((0, 3), (31, 34), (4094, 4098), (8189, 8192)):        # group edges, middle, last rows
        want = oracle.attention_exact(f16_bits(q), okv, 0, rope_np, shape.hq, shape.rd, shape.qscale, rows=(lo, hi))
        assert_close(got[lo:hi], want[lo:hi], f"prefill rows {lo}..{hi}")


def _oracle_view(oracle, layer):
    """The oracle's cache object over the bytes of a GPU-built cache (the codec's bit-exactness is tested on its own)."""
    okv = oracle.KvCache(layer.hkv, layer.hd, layer.max_ctx)
    for name, arr in layer.to_numpy().items():
        getattr(okv, name)[...] = arr.reshape(getattr(okv, name).shape)
    return okv


def test_config5_decode_batch_at_mixed_contexts(oracle):
    """Eight independent single-token decodes at 2k ... 128k, every one against the exact oracle over all its keys (the long
    ones are where the rotation by angle addition is furthest from the table); the tensor-core kernel is also compared with
    the CUDA-core kernel.  Up to 16,384 tokens the oracle encodes the cache itself; beyond, it reads the GPU-built bytes."""
    from yasakani_b200 import kv4
    shape = synth.C2
    for i, ctx in enumerate((2048, 4096, 8192, 16384, 32768, 65536, 98304, 131072)):
        small = ctx <= 16384
        layer, okv, max_ctx = _build(kv4, oracle, shape, ctx, seed=80 + i, want_oracle=small)
        if small:
            got_cache = layer.to_numpy()
            for name, want in okv.arrays().items():
                assert np.array_equal(got_cache[name].reshape(want.shape), want), f"ctx {ctx}: {name}"
        else:
            okv = _oracle_view(oracle, layer)
        rope = _rope(kv4, shape, max_ctx)
        q = synth.make_q(shape, 1, seed=80 + i)
        d_pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
        outs = {}
        for algo in (ALGO_AUTO, ALGO_SCALAR):
            kv4.set_algo(algo)
            pm, pl, pacc = kv4.attn_scratch(1, 37, shape.hq, shape.hd)
            o16 = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
            kv4.launch_decode(q.cuda(), layer, 1, d_pos, 37, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16)
            torch.cuda.synchronize()
            outs[algo] = o16.float().cpu().numpy()
        kv4.set_algo(ALGO_AUTO)
        assert kv4.device_status() == 0
        assert_close(outs[ALGO_AUTO], outs[ALGO_SCALAR], f"ctx {ctx}: tensor-core vs CUDA-core")
        want = oracle.attention_exact(f16_bits(q), okv, ctx - 1, rope.cpu().numpy(), shape.hq, shape.rd, shape.qscale)
        worst = assert_close(outs[ALGO_AUTO], want, f"ctx {ctx} vs oracle")
        print(f"decode ctx {ctx}: max abs err vs exact oracle {worst:.3e}")
        del layer, rope, okv
        torch.cuda.empty_cache()


def test_config5_eight_decodes_as_one_launch(oracle):
    """The decode batch of config 5 as ONE launch (yskn_kv4_attention_ms): eight sequences at 2k ... 128k, one row each;
    every row equals the single-sequence launch bit for bit and the exact oracle within the bar."""
    from yasakani_b200 import kv4
    shape, S = synth.C2, 19
    ctxs = (2048, 4096, 8192, 16384, 32768, 65536, 98304, 131072)
    max_ctx = 131072 + 64
    layers = []
    for i, ctx in enumerate(ctxs):
        layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
        d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        for c in range(ctx // CHUNK if ctx >= CHUNK else 1):
            n = min(CHUNK, ctx)
            k, v = synth.make_kv(shape, n, seed=(80 + i) * 1000 + c)
            d_pos.fill_(c * CHUNK)
            kv4.launch_kv_append(layer, k.cuda(), v.cuda(), d_pos, n)
        layers.append(layer)
    rope = _rope(kv4, shape, max_ctx)
    M = len(ctxs)
    q = synth.make_q(shape, M, seed=88)
    dq = q.cuda()
    slots = kv4.MsSlots(layers)
    pos = torch.tensor([c - 1 for c in ctxs], dtype=torch.int32, device="cuda")
    slot = torch.arange(M, dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, S, shape.hq, shape.hd)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_attention_ms(dq, slots, M, pos, slot, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd)
    kv4.launch_attn_combine_gqa(pm, pl, pacc, S, M, o16, shape.hq, shape.g)
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
    rope_np = rope.cpu().numpy()
    for r, ctx in enumerate(ctxs):
        d_pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
        pm1, pl1, pacc1 = kv4.attn_scratch(1, S, shape.hq, shape.hd)
        kv4.launch_attention_gqa(dq[r:r + 1].contiguous(), layers[r], 1, d_pos, S, pm1, pl1, pacc1, rope, shape.hq, shape.qscale, shape.rd)
        torch.cuda.synchronize()
        assert torch.equal(pacc[r].view(torch.int32), pacc1[0].view(torch.int32)), f"ctx {ctx}"
        if ctx <= 32768:
            want = oracle.attention_exact(f16_bits(q[r:r + 1]), _oracle_view(oracle, layers[r]), ctx - 1, rope_np, shape.hq, shape.rd, shape.qscale)
            assert_close(o16[r:r + 1].float().cpu().numpy(), want, f"ctx {ctx} vs oracle")


@pytest.mark.parametrize("form", ["workspace", "converting"])
def test_config3_verify_widths_over_32768_tokens(oracle, form):
    """16-, 32- and 64-row verify passes over a 32,768-token cache: shared rows bitwise identical; every row vs the oracle.
    Both forms of the tcgen05 kernel: over the dequantised workspace, and converting the packed cache inside the kernel."""
    from yasakani_b200 import kv4
    shape, ctx = synth.C2, 32768
    base, okv, max_ctx = _build(kv4, oracle, shape, ctx, seed=90)
    max_ctx = base.max_ctx
    rope = _rope(kv4, shape, max_ctx)
    k_new, v_new = synth.make_kv(shape, 64, seed=91)
    q = synth.make_q(shape, 64, seed=91)
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    outs = {}
    for M, splits in ((16, 37), (32, 18), (64, 12)):
        layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
        for a, b in zip(layer.tensors(), base.tensors()):
            a.copy_(b)
        kv4.launch_kv_append(layer, k_new[:M].cuda(), v_new[:M].cuda(), d_pos, M)
        pm, pl, pacc = kv4.attn_scratch(M, 7, shape.hq, shape.hd)          # same split count for every width
        o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
        kv4.launch_attention_tc(q[:M].cuda(), layer, M, d_pos, 7, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd,
                                kv4.tc_workspace(layer, M) if form == "workspace" else None)
        kv4.launch_attn_combine_gqa(pm, pl, pacc, 7, M, o16, shape.hq, shape.g)
        torch.cuda.synchronize()
        assert kv4.device_status() == 0
        outs[M] = o16.cpu()
        del splits
    b16, b32, b64 = (outs[m].view(torch.int16).numpy() for m in (16, 32, 64))
    assert np.array_equal(b16, b32[:16]) and np.array_equal(b32, b64[:32])
    oracle.append(okv, ctx, f16_bits(k_new), f16_bits(v_new))
    rope_np = rope.cpu().numpy()
    got = outs[64].float().numpy()
    # every row of the widest pass against the exact oracle, and the distribution of the error relative to the bar
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(got, want, "verify, all 64 rows")
    err = np.abs(got - want)
    ratio = err / (2e-3 + 1e-2 * np.abs(want))
    print(f"verify ({form} form) 64 rows vs 32768 tokens: max abs err {err.max():.3e}, p99 {np.percentile(err, 99):.3e}, "
          f"largest fraction of the bar {ratio.max():.3f}, p99 {np.percentile(ratio, 99):.3f}")
    assert np.percentile(ratio, 99) <= 0.5, "the bulk of the verify error should sit well inside the bar"
