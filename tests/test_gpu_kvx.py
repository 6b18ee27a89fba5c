"""Family-B row codec, step 1 on the GPU, through the C ABI: bit-exact against the CPU oracle and the known answers."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kvx_kat.npz")


def _rows(n, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, 256)) * np.exp(rng.uniform(np.log(0.05), np.log(20.0), (n, 1)))
    x[n // 3] = 0.0                                   # an all-zero row
    x[n // 2, :] = 0.0; x[n // 2, 100] = -2.5         # a one-hot row
    return x.astype(np.float32)


def test_known_answers(oracle):
    from yasakani_b200 import kvx
    g = np.load(GOLD)
    x = torch.from_numpy(g["x"]).cuda()
    assert np.array_equal(kvx.rotate(x).cpu().numpy().view(np.uint32), g["rot"].view(np.uint32))
    q, sc = kvx.encode(x)
    assert np.array_equal(q.cpu().numpy(), g["q"])
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), g["scales"].view(np.uint32))
    assert np.array_equal(kvx.decode(q, sc).cpu().numpy().view(np.uint32), g["y"].view(np.uint32))


@pytest.mark.parametrize("rows", [1, 7, 8, 1000, 65537])
def test_encode_decode_rotate_equal_the_oracle_bit_for_bit(oracle, rows):
    from yasakani_b200 import kvx
    x = _rows(max(rows, 3), seed=rows)[:rows] if rows < 3 else _rows(rows, seed=rows)
    dx = torch.from_numpy(x).cuda()
    oq, osc = oracle.kvx_encode(x)
    q, sc = kvx.encode(dx)
    assert np.array_equal(q.cpu().numpy(), oq)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), osc.view(np.uint32))
    assert np.array_equal(kvx.decode(q, sc).cpu().numpy().view(np.uint32), oracle.kvx_decode(oq, osc).view(np.uint32))
    for inv in (False, True):
        assert np.array_equal(kvx.rotate(dx, inverse=inv).cpu().numpy().view(np.uint32), oracle.kvx_rotate(x, inverse=inv).view(np.uint32))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_half_precision_rows_are_widened_exactly_and_rounded_once(oracle, dtype):
    from yasakani_b200 import kvx
    x16 = torch.from_numpy(_rows(512, seed=9)).to(dtype).cuda()
    x32 = x16.float().cpu().numpy()
    oq, osc = oracle.kvx_encode(x32)
    q, sc = kvx.encode(x16)
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(sc.cpu().numpy().view(np.uint32), osc.view(np.uint32))
    want = torch.from_numpy(oracle.kvx_decode(oq, osc)).to(dtype)          # one round-to-nearest-even of the fp32 result
    got = kvx.decode(q, sc, dtype=dtype).cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_round_trip_properties_at_cache_scale():
    # 1 Mi rows (a 262,144-token cache of 4 kv-heads): the rotation preserves the norm and decode(encode(x)) stays within
    # the quantiser's error; no oracle involved
    from yasakani_b200 import kvx
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((1 << 20, 256), generator=g, device="cuda")
    r = kvx.rotate(x)
    assert torch.allclose(r.norm(dim=1), x.norm(dim=1), rtol=1e-4)
    assert (kvx.rotate(r, inverse=True) - x).abs().max().item() < 1e-4
    q, sc = kvx.encode(x)
    assert int(q.abs().max(dim=1).values.min()) == 127
    y = kvx.decode(q, sc)
    assert ((y - x).pow(2).mean().sqrt() < 0.3 * sc.mean()).item()


def test_probe_has_the_reference_contract(oracle):
    from yasakani_b200 import kvx
    x = _rows(64, seed=21)
    q, sc, y = kvx.probe(x)
    oq, osc = oracle.kvx_encode(x)
    assert np.array_equal(q, oq) and np.array_equal(sc.view(np.uint32), osc.view(np.uint32))
    assert np.array_equal(y.view(np.uint32), oracle.kvx_decode(oq, osc).view(np.uint32))
    with pytest.raises(ValueError):
        kvx.probe(x[:3])                              # odd row count: rejected like the reference's probe (-1)


def test_bad_arguments_are_rejected():
    from yasakani_b200 import kvx
    with pytest.raises(ValueError):
        kvx.encode(torch.zeros(100, device="cuda"))
    with pytest.raises(TypeError):
        kvx.rotate(torch.zeros(256, device="cuda", dtype=torch.float16))
    q, sc = kvx.encode(torch.zeros((0, 256), device="cuda"))   # zero rows: a no-op
    assert q.shape == (0, 256) and sc.shape == (0,)


# ---------------------------------------------------------------- the attention block's row epilogue (yskn_kvx_attn_post)
POST_GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kvx_post_kat.npz")


def _bf_t(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).cuda()


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _gpu_post(kvx, d, eps, pos0, rd, max_ctx, pm=True, fill=0):
    M, nh, kvh = d["q_rows"].shape[0], d["q_rows"].shape[1], d["k_rows"].shape[1]
    k8 = torch.full((kvh, max_ctx, 256), fill, dtype=torch.int8, device="cuda"); v8 = torch.full_like(k8, fill)
    ks = torch.full((kvh, max_ctx), float(fill), device="cuda"); vs = torch.full_like(ks, float(fill))
    q16 = torch.empty((M, nh, 256), dtype=torch.bfloat16, device="cuda"); gate16 = torch.empty_like(q16)
    rope = torch.from_numpy(d["rope"]).cuda() if rd else None
    kvx.launch_attn_post(_bf_t(d["q_rows"]), _bf_t(d["k_rows"]), _bf_t(d["v_rows"]), _bf_t(d["qn_w"]), _bf_t(d["kn_w"]), eps,
                         torch.tensor([pos0], dtype=torch.int32, device="cuda"), rope, rd, q16, gate16, k8, ks, v8, vs, pm=pm)
    torch.cuda.synchronize()
    return _bits(q16), _bits(gate16), k8.cpu().numpy(), ks.cpu().numpy(), v8.cpu().numpy(), vs.cpu().numpy()


def _oracle_post(oracle, d, eps, pos0, rd, max_ctx, fill=0):
    kvh = d["k_rows"].shape[1]
    k8 = np.full((kvh, max_ctx, 256), fill, dtype=np.int8); v8 = np.full_like(k8, fill)
    ks = np.full((kvh, max_ctx), float(fill), dtype=np.float32); vs = np.full_like(ks, float(fill))
    q16, gate16 = oracle.kvx_attn_post(d["q_rows"], d["k_rows"], d["v_rows"], d["qn_w"], d["kn_w"], eps, pos0, d["rope"], rd, max_ctx, k8, ks, v8, vs)
    return q16, gate16, k8, ks, v8, vs


def _same(got, want, what):
    for g_, w_, n in zip(got, want, ("q16", "gate16", "k8", "ks", "v8", "vs")):
        a = g_.view(np.uint32) if g_.dtype == np.float32 else g_
        b = w_.view(np.uint32) if w_.dtype == np.float32 else w_
        assert np.array_equal(a, b), f"{what}: {n} differs in {int((a != b).sum())} of {a.size} elements"


def test_attn_post_known_answers():
    from yasakani_b200 import kvx
    g = np.load(POST_GOLD)
    for name, c in {"a": dict(rd=64, max_ctx=64, pos0=37, eps=1e-6), "b": dict(rd=128, max_ctx=32, pos0=5, eps=1e-5)}.items():
        d = {k_: g[f"{name}_{k_}"] for k_ in ("q_rows", "k_rows", "v_rows", "qn_w", "kn_w", "rope")}
        q16, gate16, k8, ks, v8, vs = _gpu_post(kvx, d, c["eps"], c["pos0"], c["rd"], c["max_ctx"])
        M = d["q_rows"].shape[0]; sl = slice(c["pos0"], c["pos0"] + M)
        _same((q16, gate16, k8[:, sl], ks[:, sl], v8[:, sl], vs[:, sl]),
              tuple(g[f"{name}_{k_}"] for k_ in ("q16", "gate16", "k8", "ks", "v8", "vs")), f"known answers {name}")


@pytest.mark.parametrize("M,nh,kvh,rd,pos0", [(1, 24, 4, 64, 0), (5, 24, 4, 64, 1000), (33, 8, 2, 128, 17), (7, 6, 1, 0, 3), (4, 16, 2, 256, 60),
                                              (3, 5, 3, 192, 9)])
def test_attn_post_equals_the_oracle_bit_for_bit(oracle, M, nh, kvh, rd, pos0):
    """Bit-exact in the portable-math mode; rows that are not appended keep their contents (the caches start filled with 7)."""
    from tests.helpers import post_inputs
    from yasakani_b200 import kvx
    max_ctx = pos0 + M + 11
    d = post_inputs(900 + M, M, nh, kvh, rd, max_ctx)
    _same(_gpu_post(kvx, d, 1e-6, pos0, rd, max_ctx, fill=7), _oracle_post(oracle, d, 1e-6, pos0, rd, max_ctx, fill=7), f"M {M} nh {nh} kvh {kvh} rd {rd}")


def test_attn_post_default_math_mode_is_within_one_bf16_step(oracle):
    """pm = 0 takes rsqrtf like the reference's default (an approximation: no CPU restatement); against the portable-math
    oracle the query rows may differ by one bf16 step and the INT8 payload by one count."""
    from tests.helpers import post_inputs
    from yasakani_b200 import kvx
    M, nh, kvh, rd, pos0, max_ctx = 6, 24, 4, 64, 40, 64
    d = post_inputs(77, M, nh, kvh, rd, max_ctx)
    got = _gpu_post(kvx, d, 1e-6, pos0, rd, max_ctx, pm=False)
    want = _oracle_post(oracle, d, 1e-6, pos0, rd, max_ctx)
    qg = (got[0].astype(np.uint32) << 16).view(np.float32); qw = (want[0].astype(np.uint32) << 16).view(np.float32)
    assert np.abs(qg - qw).max() <= 2.0 ** -7 * np.abs(qw).max()
    assert (got[0] == want[0]).mean() > 0.9
    assert np.abs(got[2].astype(np.int32) - want[2].astype(np.int32)).max() <= 1 and np.array_equal(got[4], want[4])


def test_attn_post_outside_the_cache_stores_no_row_and_bad_arguments_are_rejected(oracle):
    from tests.helpers import post_inputs
    from yasakani_b200 import kvx, Kv4Error
    M, nh, kvh, rd, max_ctx = 4, 4, 2, 64, 16
    d = post_inputs(5, M, nh, kvh, rd, max_ctx + M)
    d["rope"] = d["rope"][:max_ctx + M]
    got = _gpu_post(kvx, d, 1e-6, max_ctx - 2, rd, max_ctx, fill=7)             # tokens 2 and 3 fall outside
    want = _oracle_post(oracle, {**d, **{k_: d[k_][:2] for k_ in ("q_rows", "k_rows", "v_rows")}}, 1e-6, max_ctx - 2, rd, max_ctx, fill=7)
    _same(got[2:], want[2:], "cache rows")
    assert np.array_equal(got[0][:2], want[0])
    with pytest.raises(Kv4Error, match="multiple of 64"):
        _gpu_post(kvx, d, 1e-6, 0, 32, max_ctx)
