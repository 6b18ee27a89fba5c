"""Family-B row codec, step 1 (sign-Hadamard-256 + INT8 rows): the CPU oracle against its known-answer file and the
properties the transform must have."""
import os

import numpy as np

from oracle import kv4_oracle as o

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kvx_kat.npz")


def test_oracle_matches_known_answers_bit_for_bit():
    g = np.load(GOLD)
    assert np.array_equal(o.kvx_sign(), g["sign"])
    assert np.array_equal(o.kvx_rotate(g["x"]).view(np.uint32), g["rot"].view(np.uint32))
    q, sc = o.kvx_encode(g["x"])
    assert np.array_equal(q, g["q"]) and np.array_equal(sc.view(np.uint32), g["scales"].view(np.uint32))
    assert np.array_equal(o.kvx_decode(q, sc).view(np.uint32), g["y"].view(np.uint32))


def test_sign_is_the_documented_hash():
    # bit 0 of a multiply-xorshift hash of d + 1 (src/kvx_codec.cuh:28-32), restated independently in numpy
    d = np.arange(256, dtype=np.uint64) + 1
    m = np.uint64(0xFFFFFFFF)
    x = d ^ (d >> np.uint64(16)); x = (x * np.uint64(0x7feb352d)) & m
    x ^= x >> np.uint64(15); x = (x * np.uint64(0x846ca68b)) & m; x ^= x >> np.uint64(16)
    want = np.where(x & np.uint64(1), -1.0, 1.0).astype(np.float32)
    assert np.array_equal(o.kvx_sign(), want)


def test_rotation_is_orthonormal_and_inverts():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((16, 256)).astype(np.float32)
    r = o.kvx_rotate(x)
    assert np.allclose(np.linalg.norm(r, axis=1), np.linalg.norm(x, axis=1), rtol=1e-5)   # H/16 is orthonormal
    assert np.abs(o.kvx_rotate(r, inverse=True) - x).max() < 1e-5
    # against the dense Walsh-Hadamard matrix in natural order
    H = np.array([[1.0]])
    for _ in range(8):
        H = np.block([[H, H], [H, -H]])
    want = (x.astype(np.float64) * o.kvx_sign()) @ H.T / 16.0
    assert np.abs(r - want).max() < 1e-4


def test_quantiser_edges():
    z = np.zeros((2, 256), dtype=np.float32)
    q, sc = o.kvx_encode(z)
    assert not q.any() and not sc.any()
    assert not o.kvx_decode(q, sc).any()
    rng = np.random.default_rng(6)
    x = rng.standard_normal((32, 256)).astype(np.float32)
    q, sc = o.kvx_encode(x)
    assert np.abs(q.astype(np.int32)).max(axis=1).tolist() == [127] * 32          # the largest element maps to +-127
    r = o.kvx_rotate(x)
    assert np.allclose(sc, np.abs(r).max(axis=1) / np.float32(127))
    y = o.kvx_decode(q, sc)
    assert np.abs(y - x).max() < 4 * sc.max()                                     # a few quantisation steps per element
    assert np.sqrt(((y - x) ** 2).mean()) < 0.3 * sc.mean()                       # rms error of a uniform quantiser: step / sqrt(12)


# ---------------------------------------------------------------- the attention block's row epilogue (ysko_kvx_attn_post)
POST_GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kvx_post_kat.npz")
POST_CASES = {"a": dict(rd=64, max_ctx=64, pos0=37, eps=1e-6), "b": dict(rd=128, max_ctx=32, pos0=5, eps=1e-5)}


def _post_run(g, name, c):
    kvh, M = g[f"{name}_k_rows"].shape[1], g[f"{name}_q_rows"].shape[0]
    k8 = np.zeros((kvh, c["max_ctx"], 256), dtype=np.int8); v8 = np.zeros_like(k8)
    ks = np.zeros((kvh, c["max_ctx"]), dtype=np.float32); vs = np.zeros_like(ks)
    q16, gate16 = o.kvx_attn_post(g[f"{name}_q_rows"], g[f"{name}_k_rows"], g[f"{name}_v_rows"], g[f"{name}_qn_w"], g[f"{name}_kn_w"],
                                  c["eps"], c["pos0"], g[f"{name}_rope"], c["rd"], c["max_ctx"], k8, ks, v8, vs)
    return q16, gate16, k8, ks, v8, vs, M


def test_attn_post_oracle_matches_known_answers_bit_for_bit():
    g = np.load(POST_GOLD)
    for name, c in POST_CASES.items():
        q16, gate16, k8, ks, v8, vs, M = _post_run(g, name, c)
        sl = slice(c["pos0"], c["pos0"] + M)
        assert np.array_equal(q16, g[f"{name}_q16"]) and np.array_equal(gate16, g[f"{name}_gate16"])
        assert np.array_equal(k8[:, sl], g[f"{name}_k8"]) and np.array_equal(v8[:, sl], g[f"{name}_v8"])
        assert np.array_equal(ks[:, sl].view(np.uint32), g[f"{name}_ks"].view(np.uint32))
        assert np.array_equal(vs[:, sl].view(np.uint32), g[f"{name}_vs"].view(np.uint32))
        # nothing outside the appended positions is written
        k8[:, sl] = 0; v8[:, sl] = 0; ks[:, sl] = 0; vs[:, sl] = 0
        assert not k8.any() and not v8.any() and not ks.any() and not vs.any()


def _bf(x):                                   # bf16 bits -> fp32
    return (np.asarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _rbf(x):                                  # fp32 -> nearest-even bf16 -> fp32 (finite values)
    u = np.asarray(x, dtype=np.float32).view(np.uint32)
    return (((u + np.uint32(0x7fff) + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def _norm_rope_numpy(rows16, w16, eps, rope_row, rd):
    """q35_attn_post_kernel's norm + RoPE on rows [n][256] in numpy fp32 (one IEEE operation per step), written independently
    of the C oracle: shuffle-tree sum of squares per 32 channels, in-order sum of the 8 warp sums, 1/sqrt, bf16 roundings."""
    y = _bf(rows16); f = np.float32
    t = (y * y).reshape(-1, 8, 32)
    j = np.arange(32)
    for s in (16, 8, 4, 2, 1):
        t = t + t[:, :, j ^ s]
    tot = np.zeros(t.shape[0], dtype=f)
    for w in range(8):
        tot = tot + t[:, w, 0]
    r = f(1.0) / np.sqrt(tot / f(256.0) + f(eps))
    xn = _rbf((y * r[:, None]) * (f(1.0) + _bf(w16))[None, :])
    out = xn.copy()
    h = rd // 2
    if h:
        c, s = rope_row[:, 0][None, :], rope_row[:, 1][None, :]
        out[:, :h] = _rbf(_rbf(xn[:, :h] * c) + _rbf(-xn[:, h:rd] * s))
        out[:, h:rd] = _rbf(_rbf(xn[:, h:rd] * c) + _rbf(xn[:, :h] * s))
    return out


def test_attn_post_oracle_equals_an_independent_numpy_restatement():
    g = np.load(POST_GOLD)
    for name, c in POST_CASES.items():
        q16, gate16, k8, ks, v8, vs, M = _post_run(g, name, c)
        q_rows, k_rows, v_rows = g[f"{name}_q_rows"], g[f"{name}_k_rows"], g[f"{name}_v_rows"]
        assert np.array_equal(gate16, q_rows[:, :, 256:])
        for t in range(M):
            rr = g[f"{name}_rope"][c["pos0"] + t]
            xq = _norm_rope_numpy(q_rows[t, :, :256], g[f"{name}_qn_w"], c["eps"], rr, c["rd"])
            assert np.array_equal(_rbf(o.kvx_rotate(xq)).view(np.uint32) >> 16, q16[t].astype(np.uint32))
            xk = _norm_rope_numpy(k_rows[t], g[f"{name}_kn_w"], c["eps"], rr, c["rd"])
            qk, sk = o.kvx_encode(xk)
            assert np.array_equal(qk, k8[:, c["pos0"] + t]) and np.array_equal(sk.view(np.uint32), ks[:, c["pos0"] + t].view(np.uint32))
            qv, sv = o.kvx_encode(_bf(v_rows[t]))
            assert np.array_equal(qv, v8[:, c["pos0"] + t]) and np.array_equal(sv.view(np.uint32), vs[:, c["pos0"] + t].view(np.uint32))


def test_attn_post_keeps_the_query_key_product():
    """Norm and RoPE aside, rotation is orthonormal: q . k of the outputs (decoded) stays close to q . k of the un-rotated
    normed and roped rows."""
    g = np.load(POST_GOLD); name, c = "a", POST_CASES["a"]
    q16, _, k8, ks, _, _, _ = _post_run(g, name, c)
    rr = g[f"{name}_rope"][c["pos0"]]
    xq = _norm_rope_numpy(g[f"{name}_q_rows"][0, :, :256], g[f"{name}_qn_w"], c["eps"], rr, c["rd"]).astype(np.float64)
    xk = _norm_rope_numpy(g[f"{name}_k_rows"][0], g[f"{name}_kn_w"], c["eps"], rr, c["rd"]).astype(np.float64)
    want = xq[:6] @ xk[0]
    got = _bf(q16[0, :6]).astype(np.float64) @ (k8[0, c["pos0"]].astype(np.float64) * float(ks[0, c["pos0"]]))
    assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max() + 0.5
