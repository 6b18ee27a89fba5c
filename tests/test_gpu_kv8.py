"""Family-B decode attention over INT8 rows (yskn_kv8_attention / yskn_kv8_combine) against the CPU oracle.
Tolerance: max-abs 2e-3 / rel 1e-2 on the merged rows, the bar of the KV4 path."""
import numpy as np
import pytest
import torch

from tests.helpers import ATOL, RTOL, assert_close

pytestmark = pytest.mark.gpu
NH, KVH = 24, 4


def _case(oracle, ctx, M, seed, max_ctx=None, kvh=KVH, nh=NH):
    """INT8 cache of ctx + M tokens built by the row codec from seeded K/V rows; rotated, rounded queries."""
    rng = np.random.default_rng(seed)
    n = ctx + M
    max_ctx = max_ctx or ((n + 63) // 64) * 64
    k = rng.standard_normal((kvh, n, 256)).astype(np.float32) * np.exp(rng.uniform(np.log(0.5), np.log(4.0), (kvh, 1, 256))).astype(np.float32)
    v = rng.standard_normal((kvh, n, 256)).astype(np.float32)
    k8 = np.zeros((kvh, max_ctx, 256), np.int8); v8 = np.zeros_like(k8)
    ks = np.full((kvh, max_ctx), np.nan, np.float32); vs = np.full((kvh, max_ctx), np.nan, np.float32)   # rows past the context must never matter
    for h in range(kvh):
        k8[h, :n], ks[h, :n] = oracle.kvx_encode(k[h])
        v8[h, :n], vs[h, :n] = oracle.kvx_encode(v[h])
    q = oracle.kvx_rotate(rng.standard_normal((M * nh, 256)).astype(np.float32)).reshape(M, nh, 256)
    return k8, v8, ks, vs, q, max_ctx


def _run(kvx, k8, v8, ks, vs, q, ctx, M, splits, dtype, gate=None, inverse=True, nh=NH):
    dq = torch.from_numpy(q).to(dtype).cuda()
    d = [torch.from_numpy(a).cuda() for a in (k8, v8, ks, vs)]
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    pm = torch.empty((M, splits, nh), device="cuda"); pl = torch.empty_like(pm); pacc = torch.empty((M, splits, nh, 256), device="cuda")
    kvx.launch_kv8_attention(dq, *d, M, d_pos, splits, pm, pl, pacc, nh)
    o = torch.empty((M, nh, 256), dtype=dtype, device="cuda")
    kvx.launch_kv8_combine(pm, pl, pacc, splits, M, nh, o, gate=gate, inverse_rotate=inverse)
    torch.cuda.synchronize()
    return o.float().cpu().numpy(), dq.float().cpu().numpy(), (pm, pl, pacc)


@pytest.mark.parametrize("ctx,M,splits", [(0, 1, 1), (15, 1, 4), (16, 1, 1), (97, 3, 5), (2065, 1, 37), (8191, 2, 37), (5000, 1, 64)])
def test_decode_matches_exact_attention_fp16(oracle, ctx, M, splits):
    from yasakani_b200 import kvx
    k8, v8, ks, vs, q, _ = _case(oracle, ctx, M, seed=ctx + M)
    got, q16, _ = _run(kvx, k8, v8, ks, vs, q, ctx, M, splits, torch.float16, inverse=False)
    want = oracle.kv8_attention_exact(q16, k8, v8, ks, vs, ctx)
    assert_close(got, want, f"kv8 decode ctx {ctx} M {M} S {splits} (rotated basis)")
    got_r, _, _ = _run(kvx, k8, v8, ks, vs, q, ctx, M, splits, torch.float16, inverse=True)
    assert_close(got_r, oracle.kvx_rotate(want.reshape(-1, 256), inverse=True).reshape(want.shape), "after the inverse rotation")


def _run_tc(kvx, k8, v8, ks, vs, q, ctx, M, splits, dtype, nh=NH, plain_entry=False):
    dq = torch.from_numpy(q).to(dtype).cuda()
    d = [torch.from_numpy(a).cuda() for a in (k8, v8, ks, vs)]
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    pm = torch.full((M, splits, nh), float("nan"), device="cuda"); pl = torch.full_like(pm, float("nan"))
    pacc = torch.full((M, splits, nh, 256), float("nan"), device="cuda")
    (kvx.launch_kv8_attention if plain_entry else kvx.launch_kv8_attention_tc)(dq, *d, M, d_pos, splits, pm, pl, pacc, nh)
    o = torch.empty((M, nh, 256), dtype=dtype, device="cuda")
    kvx.launch_kv8_combine(pm, pl, pacc, splits, M, nh, o, inverse_rotate=False)
    torch.cuda.synchronize()
    from yasakani_b200 import kv4
    assert kv4.device_status() == 0
    assert torch.isfinite(pm).all() and torch.isfinite(pl).all() and torch.isfinite(pacc).all(), "a partial slot was not written"
    return o.float().cpu().numpy(), dq.float().cpu().numpy(), pacc


@pytest.mark.parametrize("ctx,M,splits,nh,dtype", [
    (0, 16, 1, 24, torch.float16),          # first rows of a sequence: causal inside the first tile
    (0, 100, 1, 24, torch.float16),         # several query tiles
    (200, 16, 3, 24, torch.float16),
    (1024, 64, 5, 24, torch.float16),       # verify shape, scaled down
    (4000, 32, 13, 24, torch.bfloat16),     # the reference's activation dtype
    (300, 40, 4, 32, torch.float16),        # 8 query heads per kv-head
    (500, 30, 2, 28, torch.bfloat16),       # 7 heads per kv-head: idle rows in the tile
])
def test_many_rows_on_the_tensor_core_kernel_match_exact_attention(oracle, ctx, M, splits, nh, dtype):
    from yasakani_b200 import kvx
    k8, v8, ks, vs, q, _ = _case(oracle, ctx, M, seed=100 + ctx + M, nh=nh)
    got, q16, _ = _run_tc(kvx, k8, v8, ks, vs, q, ctx, M, splits, dtype, nh=nh)
    want = oracle.kv8_attention_exact(q16, k8, v8, ks, vs, ctx)
    tol = dict(atol=ATOL + 2 ** -8, rtol=RTOL) if dtype == torch.bfloat16 else {}
    assert_close(got, want, f"kv8 rows on tcgen05 ctx {ctx} M {M} S {splits} nh {nh}", **tol)


def test_verify_widths_over_32768_int8_rows(oracle):
    """Configuration 3 on Family-B rows: 16-, 32- and 64-row passes over 32,768 cached tokens; shared rows bitwise identical
    across the widths (same split count), every row of the widest pass against the exact oracle."""
    from yasakani_b200 import kvx
    ctx, S = 32768, 9
    k8, v8, ks, vs, q, _ = _case(oracle, ctx, 64, seed=321)
    outs = {}
    for M in (16, 32, 64):
        got, q16, _ = _run_tc(kvx, k8, v8, ks, vs, q[:M], ctx, M, S, torch.bfloat16)
        outs[M] = got
    assert np.array_equal(outs[16], outs[32][:16]) and np.array_equal(outs[32], outs[64][:32])
    want = oracle.kv8_attention_exact(q16, k8, v8, ks, vs, ctx)
    assert_close(outs[64], want, "kv8 verify, all 64 rows vs 32768 tokens", atol=ATOL + 2 ** -8, rtol=RTOL)


def test_many_rows_agree_with_the_decode_kernel_and_the_plain_entry_takes_them(oracle):
    """Rows of a 12-row pass against twelve one-row decodes (the kernel pinned against the reference's own), and
    yskn_kv8_attention with more than 8 rows bit-identical with yskn_kv8_attention_tc."""
    from yasakani_b200 import kvx
    ctx, M, S = 1500, 12, 6
    k8, v8, ks, vs, q, _ = _case(oracle, ctx, M, seed=77)
    got, _, pacc_tc = _run_tc(kvx, k8, v8, ks, vs, q, ctx, M, S, torch.float16)
    _, _, pacc_plain = _run_tc(kvx, k8, v8, ks, vs, q, ctx, M, S, torch.float16, plain_entry=True)
    assert torch.equal(pacc_tc.view(torch.int32), pacc_plain.view(torch.int32))
    for r in range(M):
        one, _, _ = _run(kvx, k8, v8, ks, vs, q[r:r + 1], ctx + r, 1, S, torch.float16, inverse=False)
        assert_close(got[r:r + 1], one, f"row {r} against its own decode")


def test_bf16_queries_gate_and_roundings(oracle):
    # the reference's dtypes: bf16 q16, bf16 output, sigmoid gate with its three roundings (src/q35_kernels.cu:1421-1424)
    from yasakani_b200 import kvx
    ctx, M, S = 3000, 2, 32
    k8, v8, ks, vs, q, _ = _case(oracle, ctx, M, seed=7)
    rng = np.random.default_rng(8)
    gate = torch.from_numpy(rng.standard_normal((M, NH, 256)).astype(np.float32)).to(torch.bfloat16).cuda()
    got, q16, _ = _run(kvx, k8, v8, ks, vs, q, ctx, M, S, torch.bfloat16, gate=gate, inverse=True)
    y = oracle.kvx_rotate(oracle.kv8_attention_exact(q16, k8, v8, ks, vs, ctx).reshape(-1, 256), inverse=True).reshape(M, NH, 256)
    rbf = lambda a: torch.from_numpy(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    sg = rbf(1.0 / (1.0 + np.exp(-gate.float().cpu().numpy())))
    want = rbf(rbf(y) * sg)
    assert_close(got, want, "gated bf16 rows", atol=ATOL + 2 ** -8, rtol=RTOL)     # one bf16 ulp at |y| <= 1 on top of the bar


def test_result_does_not_depend_on_the_split_count_beyond_tolerance_and_rows_are_causal(oracle):
    from yasakani_b200 import kvx
    ctx, M = 1234, 4
    k8, v8, ks, vs, q, _ = _case(oracle, ctx, M, seed=3)
    a, q16, _ = _run(kvx, k8, v8, ks, vs, q, ctx, M, 1, torch.float16, inverse=False)
    b, _, _ = _run(kvx, k8, v8, ks, vs, q, ctx, M, 23, torch.float16, inverse=False)
    assert_close(a, b, "1 split vs 23 splits")
    # row r alone (M = 1 at position ctx + r) gives the same row: rows only see keys up to their own position
    for r in (0, 3):
        one, _, _ = _run(kvx, k8, v8, ks, vs, q[r:r + 1], ctx + r, 1, 7, torch.float16, inverse=False)
        assert_close(one[0], a[r], f"row {r} alone")


def test_empty_splits_write_neutral_partials(oracle):
    from yasakani_b200 import kvx
    k8, v8, ks, vs, q, _ = _case(oracle, 20, 1, seed=5)
    _, _, (pm, pl, pacc) = _run(kvx, k8, v8, ks, vs, q, 20, 1, 16, torch.float16)      # 2 tiles, 16 splits: 14 are empty
    assert (pm[0, 2:] <= -1e29).all() and (pl[0, 2:] == 0).all() and (pacc[0, 2:] == 0).all()
    assert torch.isfinite(pacc).all() and torch.isfinite(pl).all()


def test_bad_arguments_are_rejected(oracle):
    from yasakani_b200 import kvx
    from yasakani_b200._lib import Kv4Error
    k8, v8, ks, vs, q, _ = _case(oracle, 10, 1, seed=1)
    d = [torch.from_numpy(a).cuda() for a in (k8, v8, ks, vs)]
    dq = torch.from_numpy(q).to(torch.float16).cuda(); d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    pm = torch.empty((1, 2, 36), device="cuda"); pl = torch.empty_like(pm); pacc = torch.empty((1, 2, 36, 256), device="cuda")
    with pytest.raises(Kv4Error):
        kvx.launch_kv8_attention(dq, *d, 1, d_pos, 2, pm, pl, pacc, 36)                   # 9 query heads per kv-head
    with pytest.raises(Kv4Error):
        kvx.launch_kv8_combine(pm, pl, pacc, 65, 1, 24, torch.empty((1, 24, 256), dtype=torch.float16, device="cuda"))


def test_cache_scale_round_trip_properties():
    # 131,072 tokens: keys whose rows equal the (rotated) query of a head dominate the softmax, so the output must be that key's value row
    from yasakani_b200 import kvx
    ctx, kvh, nh = 131072, 2, 4
    g = torch.Generator(device="cuda").manual_seed(2)
    k = torch.randn((kvh * ctx, 256), generator=g, device="cuda"); v = torch.randn((kvh * ctx, 256), generator=g, device="cuda")
    hit = 77777
    qv = torch.randn((nh, 256), generator=g, device="cuda")
    for h in range(nh):
        k[(h // 2) * ctx + hit + h] = qv[h] * 40.0                         # one dominant key per head
    k8, ks = kvx.encode(k); v8, vs = kvx.encode(v)
    q = kvx.rotate(qv).to(torch.float16).reshape(1, nh, 256)
    d_pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    S = 37
    pm = torch.empty((1, S, nh), device="cuda"); pl = torch.empty_like(pm); pacc = torch.empty((1, S, nh, 256), device="cuda")
    kvx.launch_kv8_attention(q, k8.view(kvh, ctx, 256), v8.view(kvh, ctx, 256), ks.view(kvh, ctx), vs.view(kvh, ctx), 1, d_pos, S, pm, pl, pacc, nh)
    o = torch.empty((1, nh, 256), dtype=torch.float16, device="cuda")
    kvx.launch_kv8_combine(pm, pl, pacc, S, 1, nh, o, inverse_rotate=True)
    want = kvx.decode(v8, vs).view(kvh, ctx, 256)
    for h in range(nh):
        assert (o[0, h].float() - want[h // 2, hit + h]).abs().max().item() < 2e-2
