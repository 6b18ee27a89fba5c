"""GPU parity of KV4 attention (split-K partials + merge) through the C ABI against the CPU oracle.

Bar: |got - want| <= 2e-3 + 1e-2*|want| against a double-accumulated softmax over the dequantised cache.
"""
import glob
import os

import numpy as np
import pytest
import torch

from tests.helpers import ATOL, RTOL, assert_close, bits_f16, build_oracle_cache, f16_bits, gpu_append_all, gpu_attention
from yasakani_b200 import synth, ALGO_AUTO, ALGO_SCALAR, ALGO_MMA

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _setup(oracle, shape, ctx, M, seed, chunk=None):
    from yasakani_b200 import kv4
    okv, k16, v16 = build_oracle_cache(oracle, shape, ctx + M, seed=seed, chunk=chunk)
    layer = kv4.KvLayer(shape.hkv, shape.hd, okv.max_ctx).load_numpy(okv.arrays())
    q = synth.make_q(shape, M, seed=seed)
    rope_np = oracle.rope_table(okv.max_ctx, shape.theta, shape.rd) if shape.rd else None
    rope = torch.from_numpy(rope_np).cuda() if shape.rd else None
    return kv4, okv, layer, q, rope_np, rope


@pytest.fixture(autouse=True)
def _reset_algo():
    yield
    from yasakani_b200 import kv4
    kv4.set_algo(ALGO_AUTO)


CASES = [
    # shape, cached ctx, M rows, splits
    (synth.C1, 4095, 1, 32),                                     # config 1: pos 4095 -> 4,096 keys
    (synth.C1, 33, 1, 32),                                       # more splits than keys per split
    (synth.C1, 0, 1, 4),                                         # first token: one key, from the shadow
    (synth.C2, 8191, 1, 37),                                     # config 2, smallest context
    (synth.C2, 1000, 3, 16),
    (synth.C2, 31, 2, 8),                                        # only shadow keys
    (synth.Shape(8, 1, 64, 64, 1e4), 777, 2, 9),
    (synth.Shape(7, 1, 128, 128, 1e6), 500, 1, 32),              # G = 7 as in the reference's 7B instantiation
]


@pytest.mark.parametrize("algo", [ALGO_SCALAR, ALGO_AUTO])
@pytest.mark.parametrize("shape,ctx,M,splits", CASES)
def test_attention_matches_exact_oracle(oracle, shape, ctx, M, splits, algo):
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, M, seed=31, chunk=61)
    kv4.set_algo(algo)
    got, (pm, pl, pacc) = gpu_attention(kv4, layer, q, ctx, splits, rope, shape)
    assert np.isfinite(pm).all() and np.isfinite(pl).all() and np.isfinite(pacc).all(), "a partial slot was not written"
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(got, want, f"attention {shape} ctx {ctx} M {M}")


def test_combine_matches_literal_merge_with_bias_and_gate(oracle):
    shape, ctx, M, S = synth.C2, 300, 2, 11
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, M, seed=32)
    pm, pl, pacc = oracle.attention_partials(f16_bits(q), okv, ctx, S, rope_np, shape.hq, shape.rd, shape.qscale)
    g = torch.Generator().manual_seed(1)
    bv = torch.randn((shape.hkv, shape.hd), generator=g).half(); gate = torch.randn((M, shape.hq, shape.hd), generator=g).half()
    want = bits_f16(oracle.combine(pm, pl, pacc, shape.g, bv=f16_bits(bv), gate=f16_bits(gate)))
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_attn_combine_gqa(torch.from_numpy(pm).cuda(), torch.from_numpy(pl).cuda(), torch.from_numpy(pacc).cuda(), S, M, o16,
                                shape.hq, shape.g, bv=bv.cuda(), gate=gate.cuda())
    got = o16.float().cpu().numpy()
    # same formula and summation order; expf and FMA contraction may move a result by one fp16 ulp
    assert np.max(np.abs(got - want)) <= 2 ** -10 * max(1.0, float(np.abs(want).max()))
    assert np.mean(got == want) > 0.98


def test_triples_merge_like_combine(oracle):
    """local_triple + merge_triples (the multi-GPU exchange) equals combining all partials at once."""
    shape, ctx, M, S = synth.C2, 700, 1, 12
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, M, seed=33)
    pm, pl, pacc = [torch.from_numpy(a).cuda() for a in
                    oracle.attention_partials(f16_bits(q), okv, ctx, S, rope_np, shape.hq, shape.rd, shape.qscale)]
    o_all = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_attn_combine_gqa(pm, pl, pacc, S, M, o_all, shape.hq, shape.g)
    R = 3                                                        # three "ranks", 4 splits each
    triples = torch.empty((R, M, shape.hq, shape.hd + 2), dtype=torch.float32, device="cuda")
    for r in range(R):
        sl = slice(4 * r, 4 * r + 4)
        kv4.launch_local_triple(pm[:, sl].contiguous(), pl[:, sl].contiguous(), pacc[:, sl].contiguous(), 4, M, shape.hq, shape.hd, triples[r])
    o_merged = torch.empty_like(o_all)
    kv4.launch_merge_triples(triples, R, M, shape.hq, shape.g, shape.hd, o_merged)
    torch.cuda.synchronize()
    a, b = o_all.float().cpu().numpy(), o_merged.float().cpu().numpy()
    assert np.max(np.abs(a - b)) <= 2 ** -10 * max(1.0, float(np.abs(a).max()))
    assert_close(oracle.merge_triples(triples[:, 0].cpu().numpy()), oracle.attention_exact(
        f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)[0], "gpu triples vs exact", atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "kv4_kat_*.npz"))))
def test_attention_reproduces_golden_outputs(path):
    from yasakani_b200 import kv4
    z = np.load(path)
    hq, hkv, hd, rd, ctx, M, max_ctx = [int(x) for x in z["meta"]]
    shape = synth.Shape(hq, hkv, hd, rd, float(z["theta"]))
    layer = kv4.KvLayer(hkv, hd, max_ctx).load_numpy({n: z[n] for n in ("kq", "kscale", "kzero", "kshadow", "vq", "vscale", "vzero")})
    q = torch.from_numpy(z["q16"].view(np.int16)).view(torch.float16)
    got, _ = gpu_attention(kv4, layer, q, ctx, 8, torch.from_numpy(z["rope"]).cuda(), shape)
    assert_close(got, z["out"], os.path.basename(path))


def test_bf16_activations(oracle):
    shape, ctx = synth.C2, 515
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, 1, seed=34)
    qb = q.to(torch.bfloat16)                                    # values are bf16-representable by construction
    got, _ = gpu_attention(kv4, layer, qb, ctx, 16, rope, shape)
    want = oracle.attention_exact(f16_bits(qb.to(torch.float16)), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(got, want, "bf16 activations", atol=4e-3)       # bf16 output rounding: 2^-9 relative


def test_rows_of_a_wider_pass_equal_the_narrower_pass(oracle):
    """Shared rows are bitwise identical whether verified 16, 32 or 64 wide (same base position).

    Rows 0-31 sit in group ctx/32 and read it from the fp16 shadow; rows 32-63 of the 64-wide pass see that
    group already quantised by the same pass (src/attention_gqa.cu:145-146)."""
    from yasakani_b200 import kv4
    shape, ctx = synth.C2, 1024
    k, v = synth.make_kv(shape, ctx + 64, seed=35)
    q = synth.make_q(shape, 64, seed=35)
    k16, v16 = f16_bits(k), f16_bits(v)
    base = oracle.KvCache(shape.hkv, shape.hd, 1152)
    oracle.append(base, 0, k16[:ctx], v16[:ctx])
    rope_np = oracle.rope_table(base.max_ctx, shape.theta, shape.rd)
    rope = torch.from_numpy(rope_np).cuda()
    outs = {}
    for M in (16, 32, 64):
        lay = kv4.KvLayer(shape.hkv, shape.hd, base.max_ctx).load_numpy(base.arrays())
        gpu_append_all(kv4, lay, k[ctx:ctx + M], v[ctx:ctx + M], [M], pos0=ctx)      # the pass appends exactly its own rows
        outs[M], _ = gpu_attention(kv4, lay, q[:M], ctx, 13, rope, shape)
    assert np.array_equal(outs[16], outs[32][:16]) and np.array_equal(outs[32], outs[64][:32])
    oracle.append(base, ctx, k16[ctx:], v16[ctx:])
    want = oracle.attention_exact(f16_bits(q), base, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(outs[64], want, "verify M=64")


def test_host_probe_runs_and_times(oracle):
    import ctypes as C
    from yasakani_b200 import _lib
    shape, ctx = synth.C1, 600
    okv, _, _ = build_oracle_cache(oracle, shape, ctx + 1, seed=36)
    q16 = f16_bits(synth.make_q(shape, 1, seed=36))
    rope = oracle.rope_table(okv.max_ctx, shape.theta, shape.rd)
    hk = _lib.KvLayerC(*[a.ctypes.data for a in (okv.kq, okv.kscale, okv.kzero, okv.kshadow, okv.vq, okv.vscale, okv.vzero)])
    out = np.zeros((1, shape.hq, shape.hd), np.uint16); ms = np.zeros(3, np.float32)
    rc = _lib.load().yskn_kv4_attention_host(q16.ctypes.data, C.byref(hk), okv.max_ctx, 1, ctx, 8, rope.ctypes.data, shape.hkv, shape.hq,
                                             shape.hd, shape.rd, C.c_float(shape.qscale), 0, out.ctypes.data, 3, ms.ctypes.data)
    assert rc == 0, _lib.load().yskn_kv4_last_error()
    assert (ms > 0).all()
    assert_close(bits_f16(out), oracle.attention_exact(q16, okv, ctx, rope, shape.hq, shape.rd, shape.qscale), "host probe")


MMA_CASES = [
    (synth.C2, 32767, 1, 74),                                    # config 2 at 32,768 keys
    (synth.C2, 4096 + 5, 1, 37),                                 # open group of 6 tokens
    (synth.C2, 4096 + 31, 1, 148),                               # full open group, more splits than groups per split
    (synth.C2, 40, 2, 4),                                        # one int4 group + open group, two rows
    (synth.C2, 15, 1, 3),                                        # open group only, less than one tile
    (synth.C1, 4095, 1, 32),
    (synth.C1, 1234, 3, 16),
    (synth.Shape(24, 4, 256, 0, 1.0), 999, 1, 8),                # no rotary channels
    (synth.Shape(5, 1, 128, 0, 1.0), 700, 1, 8),                 # odd group size, padded heads
]


@pytest.mark.parametrize("shape,ctx,M,splits", MMA_CASES)
def test_tensor_core_decode_matches_exact_oracle(oracle, shape, ctx, M, splits):
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, M, seed=37, chunk=97)
    kv4.set_algo(ALGO_MMA)
    got, (pm, pl, pacc) = gpu_attention(kv4, layer, q, ctx, splits, rope, shape)
    assert kv4.device_status() == 0
    assert np.isfinite(pm).all() and np.isfinite(pl).all() and np.isfinite(pacc).all(), "a partial slot was not written"
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(got, want, f"mma decode {shape} ctx {ctx} M {M}")
    kv4.set_algo(ALGO_SCALAR)
    ref, _ = gpu_attention(kv4, layer, q, ctx, splits, rope, shape)
    assert_close(got, ref, "mma vs cuda-core kernel", atol=1.5e-3, rtol=1e-2)


@pytest.mark.parametrize("algo", [ALGO_SCALAR, ALGO_MMA])
@pytest.mark.parametrize("world", [2, 4])
def test_shards_merge_to_the_unsharded_result(oracle, algo, world):
    """Sequence shards on ONE GPU (separate launches, no waiting on one another): shard partials -> triples -> merge."""
    from yasakani_b200.sharded import plan_shards
    shape, ctx = synth.C2, 3000
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, 1, seed=38)
    kv4.set_algo(algo)
    k, v = synth.make_kv(shape, ctx + 1, seed=38)
    triples = torch.empty((world, 1, shape.hq, shape.hd + 2), dtype=torch.float32, device="cuda")
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    dq = q.cuda()
    for rnk in range(world):
        plan = plan_shards(ctx, world, rnk, okv.max_ctx)
        lay = kv4.KvLayer(shape.hkv, shape.hd, plan.capacity)
        a, b = plan.local_rows(0, ctx + 1)
        if b > a:
            gpu_append_all(kv4, lay, k[a:b], v[a:b], [b - a], pos0=a - plan.start)
        pm, pl, pacc = kv4.attn_scratch(1, 9, shape.hq, shape.hd)
        kv4.launch_attention_shard(dq, lay, 1, d_pos, 9, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, plan.start, plan.capacity)
        kv4.launch_local_triple(pm, pl, pacc, 9, 1, shape.hq, shape.hd, triples[rnk])
    o16 = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_merge_triples(triples, world, 1, shape.hq, shape.g, shape.hd, o16)
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(o16.float().cpu().numpy(), want, f"{world} shards")


@pytest.mark.parametrize("shape,ctx,M,splits", [(synth.C2, 9000, 1, 37), (synth.C2, 300, 2, 5), (synth.C1, 2000, 1, 16), (synth.Shape(8, 1, 64, 64, 1e4), 500, 1, 6)])
def test_fused_decode_equals_attention_plus_merge(oracle, shape, ctx, M, splits):
    """yskn_kv4_decode (one launch where covered) against the two-launch sequence, twice in a row (the arrival counters reset themselves)."""
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, M, seed=39)
    g = torch.Generator().manual_seed(2)
    bv = torch.randn((shape.hkv, shape.hd), generator=g).half().cuda(); gate = torch.randn((M, shape.hq, shape.hd), generator=g).half().cuda()
    want, _ = gpu_attention(kv4, layer, q, ctx, splits, rope, shape, bv=bv, gate=gate)
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
    for _ in range(2):
        o16 = torch.full((M, shape.hq, shape.hd), float("nan"), dtype=torch.float16, device="cuda")
        kv4.launch_decode(q.cuda(), layer, M, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, bv=bv, gate=gate)
        torch.cuda.synchronize()
        assert kv4.device_status() == 0
        got = o16.float().cpu().numpy()
        assert np.max(np.abs(got - want)) <= 2 ** -10 * max(1.0, float(np.abs(want).max()))      # same formula; expf/FMA may move one fp16 ulp


@pytest.mark.parametrize("world", [1, 2, 3])
def test_peer_exchange_on_one_gpu_matches_the_gathered_merge(oracle, world):
    """push_triple / merge_pushed with all 'ranks' in one process on one GPU (every push is launched before any merge,
    so no kernel waits for a later launch), three steps in a row to exercise both halves of the exchange buffers."""
    from yasakani_b200.sharded import plan_shards
    shape, ctx = synth.C2, 2500
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, 1, seed=40)
    k, v = synth.make_kv(shape, ctx + 1, seed=40)
    bufs = [torch.zeros((kv4.exchange_bytes(world, 1, shape.hq, shape.hd) + 3) // 4, dtype=torch.float32, device="cuda") for _ in range(world)]
    xs = [kv4.peer_exchange([b.data_ptr() for b in bufs], rnk) for rnk in range(world)]
    lays, plans = [], []
    for rnk in range(world):
        plan = plan_shards(ctx, world, rnk, okv.max_ctx)
        lay = kv4.KvLayer(shape.hkv, shape.hd, plan.capacity)
        a, b = plan.local_rows(0, ctx + 1)
        if b > a:
            gpu_append_all(kv4, lay, k[a:b], v[a:b], [b - a], pos0=a - plan.start)
        lays.append(lay); plans.append(plan)
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    dq = q.cuda()
    for step in range(3):
        scratch = [kv4.attn_scratch(1, 9, shape.hq, shape.hd) for _ in range(world)]
        for rnk in range(world):
            pm, pl, pacc = scratch[rnk]
            kv4.launch_attention_shard(dq, lays[rnk], 1, d_pos, 9, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, plans[rnk].start, plans[rnk].capacity)
            kv4.launch_push_triple(pm, pl, pacc, 9, 1, shape.hq, shape.hd, xs[rnk])
        for rnk in range(world):
            o16 = torch.full((1, shape.hq, shape.hd), float("nan"), dtype=torch.float16, device="cuda")
            kv4.launch_merge_pushed(xs[rnk], 1, shape.hq, shape.g, shape.hd, o16)
            torch.cuda.synchronize()
            assert kv4.device_status() == 0
            assert_close(o16.float().cpu().numpy(), want, f"step {step} rank {rnk} of {world}")


@pytest.mark.parametrize("world", [1, 2, 3])
def test_fused_exchange_merge_on_one_gpu(oracle, world):
    """yskn_kv4_exchange_merge (fold + push + wait + merge in one launch).  On one GPU the other 'ranks' push first with the
    two-launch form (same buffer protocol), so the fused kernel finds their arrivals and never waits for a later launch;
    the rank that runs fused rotates over three steps, the others close their step with merge_pushed."""
    from yasakani_b200.sharded import plan_shards
    shape, ctx = synth.C2, 2500
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, 1, seed=41)
    k, v = synth.make_kv(shape, ctx + 1, seed=41)
    bufs = [torch.zeros((kv4.exchange_bytes(world, 1, shape.hq, shape.hd) + 3) // 4, dtype=torch.float32, device="cuda") for _ in range(world)]
    xs = [kv4.peer_exchange([b.data_ptr() for b in bufs], rnk) for rnk in range(world)]
    lays, plans = [], []
    for rnk in range(world):
        plan = plan_shards(ctx, world, rnk, okv.max_ctx)
        lay = kv4.KvLayer(shape.hkv, shape.hd, plan.capacity)
        a, b = plan.local_rows(0, ctx + 1)
        if b > a:
            gpu_append_all(kv4, lay, k[a:b], v[a:b], [b - a], pos0=a - plan.start)
        lays.append(lay); plans.append(plan)
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    dq = q.cuda()
    for step in range(3):
        fused_rank = step % world
        scratch = [kv4.attn_scratch(1, 9, shape.hq, shape.hd) for _ in range(world)]
        outs = [torch.full((1, shape.hq, shape.hd), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
        for rnk in range(world):
            pm, pl, pacc = scratch[rnk]
            kv4.launch_attention_shard(dq, lays[rnk], 1, d_pos, 9, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, plans[rnk].start, plans[rnk].capacity)
            if rnk != fused_rank:
                kv4.launch_push_triple(pm, pl, pacc, 9, 1, shape.hq, shape.hd, xs[rnk])
        pm, pl, pacc = scratch[fused_rank]
        kv4.launch_exchange_merge(pm, pl, pacc, 9, 1, shape.hq, shape.g, shape.hd, xs[fused_rank], outs[fused_rank])
        for rnk in range(world):
            if rnk != fused_rank:
                kv4.launch_merge_pushed(xs[rnk], 1, shape.hq, shape.g, shape.hd, outs[rnk])
        torch.cuda.synchronize()
        assert kv4.device_status() == 0
        for rnk in range(world):
            assert_close(outs[rnk].float().cpu().numpy(), want, f"step {step} rank {rnk} of {world}")
        assert torch.equal(outs[fused_rank], outs[(fused_rank + 1) % world])      # same triples, same merge order: same bits


def test_fused_exchange_merge_rejects_grids_that_may_not_be_resident():
    from yasakani_b200 import kv4
    from yasakani_b200._lib import Kv4Error
    shape = synth.C2
    M = 8                                                     # 24 heads x 8 rows = 192 blocks
    buf = torch.zeros((kv4.exchange_bytes(1, M, shape.hq, shape.hd) + 3) // 4, dtype=torch.float32, device="cuda")
    x = kv4.peer_exchange([buf.data_ptr()], 0)
    pm, pl, pacc = kv4.attn_scratch(M, 4, shape.hq, shape.hd)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    with pytest.raises(Kv4Error):
        kv4.launch_exchange_merge(pm, pl, pacc, 4, M, shape.hq, shape.g, shape.hd, x, o16)


def test_withheld_push_runs_the_bounded_wait_out_and_the_next_step_works(oracle):
    """A host-made failure: in a world of two (both 'ranks' on this GPU) rank 1 never pushes its triple.  With a short poll
    limit rank 0's merge must return by itself, leave o16 untouched, and report device status 7; after every exchange
    buffer is zero-filled again (the documented recovery) a normal step gives the right answer.  Nothing faults or spins
    without a bound."""
    from yasakani_b200.sharded import plan_shards
    shape, ctx, world = synth.C2, 1500, 2
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, 1, seed=43)
    k, v = synth.make_kv(shape, ctx + 1, seed=43)
    bufs = [torch.zeros((kv4.exchange_bytes(world, 1, shape.hq, shape.hd) + 3) // 4, dtype=torch.float32, device="cuda") for _ in range(world)]
    xs = [kv4.peer_exchange([b.data_ptr() for b in bufs], rnk) for rnk in range(world)]
    lays, plans = [], []
    for rnk in range(world):
        plan = plan_shards(ctx, world, rnk, okv.max_ctx)
        lay = kv4.KvLayer(shape.hkv, shape.hd, plan.capacity)
        a, b = plan.local_rows(0, ctx + 1)
        gpu_append_all(kv4, lay, k[a:b], v[a:b], [b - a], pos0=a - plan.start)
        lays.append(lay); plans.append(plan)
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    dq = q.cuda()

    def shard_partials(rnk):
        pm, pl, pacc = kv4.attn_scratch(1, 9, shape.hq, shape.hd)
        kv4.launch_attention_shard(dq, lays[rnk], 1, d_pos, 9, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, plans[rnk].start, plans[rnk].capacity)
        return pm, pl, pacc

    assert kv4.device_status() == 0
    kv4.set_peer_wait_polls(2000)                                  # about 0.2 ms instead of half a second
    try:
        kv4.launch_push_triple(*shard_partials(0), 9, 1, shape.hq, shape.hd, xs[0])      # rank 1 withholds its push
        o16 = torch.full((1, shape.hq, shape.hd), 7.0, dtype=torch.float16, device="cuda")
        kv4.launch_merge_pushed(xs[0], 1, shape.hq, shape.g, shape.hd, o16)
        torch.cuda.synchronize()                                   # returns: the wait gave up
        assert kv4.device_status() == 7
        assert kv4.device_status() == 0                            # reading clears it
        assert bool((o16 == 7.0).all())                            # no row was written from incomplete triples
    finally:
        kv4.set_peer_wait_polls(0)
    for b in bufs:                                                 # recovery: all ranks stopped, buffers cleared
        b.zero_()
    outs = []
    for rnk in range(world):
        kv4.launch_push_triple(*shard_partials(rnk), 9, 1, shape.hq, shape.hd, xs[rnk])
    for rnk in range(world):
        o = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
        kv4.launch_merge_pushed(xs[rnk], 1, shape.hq, shape.g, shape.hd, o)
        outs.append(o)
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
    for rnk in range(world):
        assert_close(outs[rnk].float().cpu().numpy(), want, f"rank {rnk} after recovery")


@pytest.mark.parametrize("shape,ctx,M", [(synth.C2, 9000, 1), (synth.C2, 5000, 3), (synth.C1, 700, 2), (synth.C2, 20, 1)])
def test_early_prefetch_changes_no_bit(oracle, shape, ctx, M):
    """The `early` promise of yskn_kv4_attn_ext (reads of *d_pos and of rows below it ahead of griddepcontrol.wait) only
    moves loads in time: partials and output are bit-identical with and without it, also for rows after the first, whose
    newest groups are written by the pass itself and must not be read early."""
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, ctx, M, seed=47)
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    dq = q.cuda()
    res = []
    for ext in (None, kv4.attn_ext(early=True)):
        pm, pl, pacc = kv4.attn_scratch(M, 11, shape.hq, shape.hd)
        o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
        for _ in range(2):                                       # back to back, so the second launch really overlaps the first merge
            kv4.launch_decode(dq, layer, M, d_pos, 11, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, ext=ext)
        torch.cuda.synchronize()
        assert kv4.device_status() == 0
        res.append((pm.cpu(), pl.cpu(), pacc.cpu(), o16.cpu()))
    for a, b in zip(*res):
        assert torch.equal(a.view(torch.int32) if a.dtype == torch.float32 else a.view(torch.int16),
                           b.view(torch.int32) if b.dtype == torch.float32 else b.view(torch.int16))
    want = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(res[1][3].float().numpy(), want, "early launch vs oracle")


@pytest.mark.parametrize("shape,base", [(synth.C2, 777), (synth.C1, 95)])
def test_tree_verify_rows_with_depth_table_and_per_row_split_counts(oracle, shape, base):
    """The extras of the 27B engine's argument set (src/q35.hpp:126-130,136; use at src/q35_atx.cu:111-119): rows of one pass
    with different visible ranges.  Row r sits at depth wk[r]: it sees the cached keys below *d_pos + wk[r] and its own key,
    stored in slot *d_pos + r.  Rows that see fewer than long_len keys use splits_short splits; their other slots are empty."""
    M, S, S_short = 8, 16, 5
    wk_host = np.array([0, 1, 2, 3, 3, 3, 4, 4], dtype=np.uint8)          # a chain of four, then alternatives at depths 3 and 4
    kv4, okv, layer, q, rope_np, rope = _setup(oracle, shape, base, M, seed=53)
    wk = torch.from_numpy(wk_host).cuda()
    long_len = base + 4                                                    # rows at depth 0..2 are "short"
    ext = kv4.attn_ext(splits_short=S_short, long_len=long_len, wk=wk)
    d_pos = torch.tensor([base], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, S, shape.hq, shape.hd)
    pm.fill_(float("nan")); pl.fill_(float("nan")); pacc.fill_(float("nan"))
    kv4.launch_attention_gqa(q.cuda(), layer, M, d_pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, ext=ext)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_attn_combine_gqa(pm, pl, pacc, S, M, o16, shape.hq, shape.g)
    torch.cuda.synchronize()
    assert torch.isfinite(pm).all() and torch.isfinite(pacc).all(), "a partial slot was not written"
    want = oracle.attention_exact(f16_bits(q), okv, base, rope_np, shape.hq, shape.rd, shape.qscale, wk=wk_host)
    assert_close(o16.float().cpu().numpy(), want, "tree verify")
    plain = oracle.attention_exact(f16_bits(q), okv, base, rope_np, shape.hq, shape.rd, shape.qscale)
    assert np.abs(plain[4:] - want[4:]).max() > 1e-3                       # the table really changes what rows 4..7 see
    pmh = pm.cpu().numpy()
    for r in range(M):
        short = base + int(wk_host[r]) + 1 < long_len
        assert (pmh[r, S_short:] <= -1e29).all() == short, f"row {r}: split count"
    # the same pass through the fused decode entry, and the rejection on the tensor-core-only setting
    o2 = torch.empty_like(o16)
    kv4.launch_decode(q.cuda(), layer, M, d_pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o2, ext=ext)
    torch.cuda.synchronize()
    assert torch.equal(o2, o16)
    from yasakani_b200._lib import Kv4Error
    kv4.set_algo(ALGO_MMA)
    with pytest.raises(Kv4Error):
        kv4.launch_attention_gqa(q.cuda(), layer, M, d_pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, ext=ext)


def test_rows_of_several_sequences_in_one_launch(oracle):
    """yskn_kv4_attention_ms: five rows from three sequences (one with two consecutive rows, as a verify pass has) in ONE
    launch; every row equals, bit for bit, the single-sequence launch of that row, and the exact oracle within the bar."""
    from yasakani_b200 import kv4
    shape, max_ctx, S = synth.C2, 5184, 13
    ctxs = [300, 2100, 5000]
    layers, okvs = [], []
    for i, ctx in enumerate(ctxs):
        okv, _, _ = build_oracle_cache(oracle, shape, ctx + 2, seed=60 + i, max_ctx=max_ctx)
        layers.append(kv4.KvLayer(shape.hkv, shape.hd, max_ctx).load_numpy(okv.arrays())); okvs.append(okv)
    rope_np = oracle.rope_table(max_ctx, shape.theta, shape.rd)
    rope = torch.from_numpy(rope_np).cuda()
    rows = [(0, ctxs[0]), (2, ctxs[2]), (2, ctxs[2] + 1), (1, ctxs[1]), (0, ctxs[0] + 1)]          # (slot, position), interleaved on purpose
    M = len(rows)
    q = synth.make_q(shape, M, seed=66)
    dq = q.cuda()
    slots = kv4.MsSlots(layers)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32, device="cuda")
    slot = torch.tensor([s for s, _ in rows], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, S, shape.hq, shape.hd)
    pm.fill_(float("nan")); pl.fill_(float("nan")); pacc.fill_(float("nan"))
    kv4.launch_attention_ms(dq, slots, M, pos, slot, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd)
    o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_attn_combine_gqa(pm, pl, pacc, S, M, o16, shape.hq, shape.g)
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
    assert torch.isfinite(pm).all() and torch.isfinite(pacc).all(), "a partial slot was not written"
    for r, (s, p) in enumerate(rows):
        d_pos = torch.tensor([p], dtype=torch.int32, device="cuda")
        pm1, pl1, pacc1 = kv4.attn_scratch(1, S, shape.hq, shape.hd)
        kv4.launch_attention_gqa(dq[r:r + 1].contiguous(), layers[s], 1, d_pos, S, pm1, pl1, pacc1, rope, shape.hq, shape.qscale, shape.rd)
        torch.cuda.synchronize()
        assert torch.equal(pacc[r].view(torch.int32), pacc1[0].view(torch.int32)) and torch.equal(pm[r].view(torch.int32), pm1[0].view(torch.int32)), f"row {r}"
        want = oracle.attention_exact(f16_bits(q[r:r + 1]), okvs[s], p, rope_np, shape.hq, shape.rd, shape.qscale)
        assert_close(o16[r:r + 1].float().cpu().numpy(), want, f"row {r} (slot {s}, position {p})")
