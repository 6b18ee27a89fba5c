"""GPU parity of the tcgen05 multi-row attention (verify pass, causal prefill) through the C ABI."""
import numpy as np
import pytest
import torch

from tests.helpers import assert_close, f16_bits, gpu_append_all
from yasakani_b200 import synth

pytestmark = pytest.mark.gpu


def _run_tc(kv4, oracle, shape, ctx, M, splits, seed, prefill=False, fused=False):
    """Cache of ctx tokens, then one pass appends M rows and attends with them. Returns (got, want).
    fused: no workspace, the kernel converts the packed cache itself."""
    k, v = synth.make_kv(shape, ctx + M, seed=seed)
    q = synth.make_q(shape, M, seed=seed)
    max_ctx = ((ctx + M + 127) // 64) * 64
    layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
    okv = oracle.KvCache(shape.hkv, shape.hd, max_ctx)
    k16, v16 = f16_bits(k), f16_bits(v)
    if ctx:
        gpu_append_all(kv4, layer, k[:ctx], v[:ctx], [ctx])
        oracle.append(okv, 0, k16[:ctx], v16[:ctx])
    gpu_append_all(kv4, layer, k[ctx:], v[ctx:], [M], pos0=ctx)
    oracle.append(okv, ctx, k16[ctx:], v16[ctx:])
    rope_np = oracle.rope_table(max_ctx, shape.theta, shape.rd) if shape.rd else None
    rope = torch.from_numpy(rope_np).cuda() if shape.rd else None
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
    pm.fill_(float("nan")); pl.fill_(float("nan")); pacc.fill_(float("nan"))
    ws = None if fused else kv4.tc_workspace(layer, M)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    if prefill:
        kv4.launch_attention_prefill_tc(q.cuda(), layer, M, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, ws)
    else:
        kv4.launch_attention_tc(q.cuda(), layer, M, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, ws)
        kv4.launch_attn_combine_gqa(pm, pl, pacc, splits, M, o16, shape.hq, shape.g)
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
    if not (prefill and splits == 1):                 # a one-split prefill finishes its rows in the kernel and writes no partials
        assert torch.isfinite(pm).all() and torch.isfinite(pl).all() and torch.isfinite(pacc).all(), "a partial slot was not written"
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    return o16.float().cpu().numpy(), want


TC_CASES = [
    # shape, cached ctx, M rows, splits
    (synth.C2, 0, 16, 1),                 # first rows of a sequence: only shadow keys, causal inside the tile
    (synth.C2, 0, 100, 1),                # several query tiles, groups complete inside the pass
    (synth.C2, 200, 16, 3),               # base not on a group boundary
    (synth.C2, 1024, 64, 5),              # verify shape (scaled down): rows 32-63 see group 32 already as int4
    (synth.C2, 4000, 32, 13),
    (synth.C1, 300, 40, 4),               # hd 128, G = 8: 16 tokens per tile
    (synth.Shape(28, 4, 128, 128, 1e6), 500, 30, 2),     # G = 7: 18 tokens per tile, 2 idle rows
    (synth.Shape(24, 4, 256, 0, 1.0), 333, 20, 2),       # no rotary channels
    (synth.Shape(24, 4, 256, 32, 1e4), 700, 20, 3),      # narrow rotary parts: two and one word pairs per key
    (synth.Shape(24, 4, 256, 16, 1e4), 260, 12, 2),
    (synth.Shape(24, 4, 256, 128, 1e4), 450, 24, 2),     # a wide rotary part: its items are converted one after the other
]


@pytest.mark.parametrize("fused", [False, True], ids=["workspace", "fused"])
@pytest.mark.parametrize("shape,ctx,M,splits", TC_CASES)
def test_tc_attention_matches_exact_oracle(oracle, shape, ctx, M, splits, fused):
    from yasakani_b200 import kv4
    got, want = _run_tc(kv4, oracle, shape, ctx, M, splits, seed=51, fused=fused)
    assert_close(got, want, f"tc attention {shape} ctx {ctx} M {M} fused {fused}")


@pytest.mark.parametrize("fused", [False, True], ids=["workspace", "fused"])
def test_tc_prefill_merges_in_one_call(oracle, fused):
    from yasakani_b200 import kv4
    got, want = _run_tc(kv4, oracle, synth.C2, 0, 700, 1, seed=52, prefill=True, fused=fused)
    assert_close(got, want, "tc prefill 700 rows")


@pytest.mark.parametrize("fused", [False, True], ids=["workspace", "fused"])
def test_tc_rows_do_not_depend_on_pass_width(oracle, fused):
    """16-, 32- and 64-row passes over the same base give bitwise identical shared rows (config 3, scaled down)."""
    from yasakani_b200 import kv4
    shape, ctx = synth.C2, 2048
    outs = {}
    for M in (16, 32, 64):
        # identical first rows: the generator is seeded per call and M only extends the stream
        k, v = synth.make_kv(shape, ctx + 64, seed=53)
        q = synth.make_q(shape, 64, seed=53)
        layer = kv4.KvLayer(shape.hkv, shape.hd, 2304)
        gpu_append_all(kv4, layer, k[:ctx], v[:ctx], [ctx])
        gpu_append_all(kv4, layer, k[ctx:ctx + M], v[ctx:ctx + M], [M], pos0=ctx)
        rope = torch.empty((2304, shape.rd // 2, 2), dtype=torch.float32, device="cuda")
        kv4.launch_rope_table_g(rope, 2304, shape.theta, shape.rd)
        d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
        pm, pl, pacc = kv4.attn_scratch(M, 7, shape.hq, shape.hd)
        o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
        kv4.launch_attention_tc(q[:M].cuda(), layer, M, d_pos, 7, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd,
                                None if fused else kv4.tc_workspace(layer, M))
        kv4.launch_attn_combine_gqa(pm, pl, pacc, 7, M, o16, shape.hq, shape.g)
        torch.cuda.synchronize()
        outs[M] = o16.cpu().view(torch.int16).numpy()
    assert np.array_equal(outs[16], outs[32][:16]) and np.array_equal(outs[32], outs[64][:32])


@pytest.mark.parametrize("form", ["workspace", "fused"])
@pytest.mark.parametrize("splits,M", [(1, 24), (4, 24), (1, 150), (3, 150)])
def test_tc_takes_bf16_activations(oracle, splits, M, form):
    """Both forms stage bf16 queries as fp16 operand rows themselves (the converter warps, or the softmax warps in the
    workspace form) and write bf16 rows (what the 27B engine passes); compared with the exact oracle on the same
    (bf16-representable) queries.  150 rows: several query tiles per head, the last one ragged."""
    from yasakani_b200 import kv4
    shape, ctx = synth.C2, 900
    k, v = synth.make_kv(shape, ctx + M, seed=81)
    q = synth.make_q(shape, M, seed=81).bfloat16()
    max_ctx = ((ctx + M + 127) // 64) * 64
    layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
    okv = oracle.KvCache(shape.hkv, shape.hd, max_ctx)
    gpu_append_all(kv4, layer, k, v, [ctx, M])
    oracle.append(okv, 0, f16_bits(k[:ctx]), f16_bits(v[:ctx])); oracle.append(okv, ctx, f16_bits(k[ctx:]), f16_bits(v[ctx:]))
    rope_np = oracle.rope_table(max_ctx, shape.theta, shape.rd); rope = torch.from_numpy(rope_np).cuda()
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.bfloat16, device="cuda")
    kv4.launch_attention_prefill_tc(q.cuda(), layer, M, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16,
                                    kv4.tc_workspace(layer, M) if form == "workspace" else None)
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
    want = oracle.attention_exact(f16_bits(q.float().half()), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    got = o16.float().cpu().numpy()
    err = np.abs(got - want)
    assert (err <= 2e-3 + 1e-2 * np.abs(want)).all(), f"bf16 pass ({form} form): max err {err.max():.3e}"
    if form == "workspace" and M > 64 and splits > 1:            # the plain entry takes a lent workspace for bf16 rows too
        pm2, pl2, pacc2 = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
        lent = kv4.tc_workspace(layer, M)
        kv4.set_tc_workspace(lent)
        try:
            kv4.launch_attention_gqa(q.cuda(), layer, M, d_pos, splits, pm2, pl2, pacc2, rope, shape.hq, shape.qscale, shape.rd)
            torch.cuda.synchronize()
        finally:
            kv4.set_tc_workspace(None)
        assert torch.equal(pacc2.view(torch.int32), pacc.view(torch.int32))


def test_tc_rejects_what_it_does_not_cover():
    from yasakani_b200 import kv4, Kv4Error
    layer = kv4.KvLayer(4, 256, 128)
    q = torch.zeros((16, 24, 256), dtype=torch.float16, device="cuda")
    d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(16, 1, 24, 256)
    with pytest.raises(Kv4Error, match="hd 128/256"):          # a rotary width that is not a whole number of 8-channel words per half
        kv4.launch_attention_tc(q, layer, 16, d_pos, 1, pm, pl, pacc, torch.zeros((128, 24), device="cuda"), 24, 0.0625, 24, kv4.tc_workspace(layer, 16))
    with pytest.raises(Kv4Error, match="workspace of"):
        kv4.launch_attention_tc(q, layer, 16, d_pos, 1, pm, pl, pacc, None, 24, 0.0625, 0, torch.empty(1024, dtype=torch.uint8, device="cuda"))


def test_tc_workspace_kept_across_passes_gives_the_same_bits(oracle):
    """Two verify passes on one cache: the second reuses the workspace of the first (valid_tokens = tokens the workspace
    already holds) and must equal a pass that dequantises everything again, bit for bit, and the oracle within the bar.
    The first pass ends inside a group, so the second has to rewrite that group once its last token has arrived."""
    from yasakani_b200 import kv4
    shape, ctx, M1, M2, splits = synth.C2, 1000, 20, 24, 4
    n = ctx + M1 + M2
    k, v = synth.make_kv(shape, n, seed=61)
    max_ctx = ((n + 127) // 64) * 64
    layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
    okv = oracle.KvCache(shape.hkv, shape.hd, max_ctx)
    gpu_append_all(kv4, layer, k[:ctx + M1], v[:ctx + M1], [ctx, M1])
    rope_np = oracle.rope_table(max_ctx, shape.theta, shape.rd)
    rope = torch.from_numpy(rope_np).cuda()
    ws = kv4.tc_workspace(layer, max(M1, M2))
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")

    def run(q, M, valid, workspace):
        pm, pl, pacc = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
        o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
        kv4.launch_attention_prefill_tc(q.cuda(), layer, M, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, workspace,
                                        valid_tokens=valid)
        torch.cuda.synchronize()
        assert kv4.device_status() == 0
        return o16

    run(synth.make_q(shape, M1, seed=62), M1, 0, ws)                       # pass 1 fills the workspace for tokens [0, ctx + M1)
    gpu_append_all(kv4, layer, k[ctx + M1:], v[ctx + M1:], [M2], pos0=ctx + M1)
    d_pos.fill_(ctx + M1)
    q2 = synth.make_q(shape, M2, seed=63)
    kept = run(q2, M2, ctx + M1, ws)                                       # pass 2 on the kept workspace
    fresh = run(q2, M2, 0, kv4.tc_workspace(layer, M2))                    # the same pass from scratch
    assert torch.equal(kept, fresh)
    oracle.append(okv, 0, f16_bits(k), f16_bits(v))
    want = oracle.attention_exact(f16_bits(q2), okv, ctx + M1, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(kept.float().cpu().numpy(), want, "second pass on a kept workspace")


def test_plain_entries_take_the_tensor_core_kernel_for_wide_passes(oracle):
    """yskn_kv4_attention with more than 8 rows runs the tcgen05 kernel: the form that converts the packed cache itself
    (bit-identical with yskn_kv4_attention_tc without a workspace), and for passes of more than 64 rows the workspace form
    (bit-identical with yskn_kv4_attention_tc at valid_tokens = 0) while a workspace is lent."""
    from yasakani_b200 import kv4
    shape, ctx, S = synth.C2, 1500, 5
    for M in (32, 80):
        k, v = synth.make_kv(shape, ctx + M, seed=71)
        q = synth.make_q(shape, M, seed=71).cuda()
        max_ctx = ((ctx + M + 127) // 64) * 64
        layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
        okv = oracle.KvCache(shape.hkv, shape.hd, max_ctx)
        gpu_append_all(kv4, layer, k, v, [ctx, M])
        oracle.append(okv, 0, f16_bits(k[:ctx]), f16_bits(v[:ctx])); oracle.append(okv, ctx, f16_bits(k[ctx:]), f16_bits(v[ctx:]))
        rope_np = oracle.rope_table(max_ctx, shape.theta, shape.rd); rope = torch.from_numpy(rope_np).cuda()
        d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")

        def run(fn):
            pm, pl, pacc = kv4.attn_scratch(M, S, shape.hq, shape.hd)
            fn(pm, pl, pacc)
            o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
            kv4.launch_attn_combine_gqa(pm, pl, pacc, S, M, o16, shape.hq, shape.g)
            torch.cuda.synchronize()
            return pacc.clone(), o16

        plain = lambda pm, pl, pacc: kv4.launch_attention_gqa(q, layer, M, d_pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd)
        ws = kv4.tc_workspace(layer, M)
        with_ws = lambda pm, pl, pacc: kv4.launch_attention_tc(q, layer, M, d_pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, ws)
        fused = lambda pm, pl, pacc: kv4.launch_attention_tc(q, layer, M, d_pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, None)
        pacc_plain, o_plain = run(plain)
        pacc_fused, _ = run(fused)
        pacc_ws, o_ws = run(with_ws)
        assert torch.equal(pacc_plain.view(torch.int32), pacc_fused.view(torch.int32))
        lent = kv4.tc_workspace(layer, M)
        kv4.set_tc_workspace(lent)
        try:
            pacc_lent, o_lent = run(plain)
        finally:
            kv4.set_tc_workspace(None)
        assert torch.equal(pacc_lent.view(torch.int32), (pacc_ws if M > 64 else pacc_fused).view(torch.int32))
        assert kv4.device_status() == 0
        want = oracle.attention_exact(f16_bits(q.cpu()), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
        assert_close(o_plain.float().cpu().numpy(), want, f"wide pass ({M} rows) through the plain entry")
        assert_close(o_lent.float().cpu().numpy(), want, f"wide pass ({M} rows) through the plain entry, workspace lent")
