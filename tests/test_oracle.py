"""CPU tests of the oracle: scalar conversions, codec rules, golden files, attention consistency.

The reference holds no golden vectors for this path; these tests cross-check the C restatement against an
independent numpy restatement of the same source lines and against the committed known-answer files.
"""
import glob
import os

import numpy as np
import pytest

from tests.helpers import ATOL, RTOL, assert_close, bits_f16, build_oracle_cache, f16_bits
from yasakani_b200 import synth

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_f16_conversions_match_ieee(oracle):
    L = oracle.lib()
    # every fp16 bit pattern round-trips exactly
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    got = np.array([L.ysko_f16_to_f32(int(h)) for h in allh], np.float32)
    fin = np.isfinite(ref)
    assert np.array_equal(got[fin], ref[fin]) and np.all(np.isnan(got[~fin]) == np.isnan(ref[~fin]))
    # fp32 -> fp16 RNE on random values, ties, subnormals and overflow edges
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 20000),
                        (ref[fin][:-1] + ref[fin][1:]) / 2,                        # exact ties between neighbours
                        np.array([65504, 65519.9, 65520, 7e4, 5.96e-8, 2.98e-8, 2.9802322e-8, 3e-8, 0.0, -0.0], np.float32)])
    x = x.astype(np.float32)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = np.array([L.ysko_f32_to_f16(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, want)


def np_quant(v, lo, hi):
    """q = rne((v-lo) * (15/(hi-lo))) clamped, fp32 steps (src/attention_gqa.cu:149-152)."""
    d = (hi - lo).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(hi > lo, np.float32(15.0) / d, np.float32(0.0)).astype(np.float32)
    q = np.rint(((v - lo).astype(np.float32) * inv).astype(np.float32)).astype(np.int32)
    return np.clip(q, 0, 15), (d / np.float32(15.0)).astype(np.float32)


@pytest.mark.parametrize("shape,ctx,chunk", [(synth.C1, 200, 37), (synth.C2, 131, 1), (synth.Shape(4, 1, 64, 64, 1e4), 96, 96)])
def test_codec_matches_numpy_restatement(oracle, shape, ctx, chunk):
    kv, k16, v16 = build_oracle_cache(oracle, shape, ctx, seed=11, chunk=chunk)
    k = bits_f16(k16); v = bits_f16(v16)                                  # [ctx][hkv][hd]
    # V: per (token, head)
    lo = v.min(-1, keepdims=True); hi = v.max(-1, keepdims=True)
    q, sc = np_quant(v, lo, hi)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)       # even channel in the low nibble
    assert np.array_equal(kv.vq[:, :ctx], packed.transpose(1, 0, 2))
    assert np.array_equal(kv.vscale[:, :ctx], sc[..., 0].astype(np.float16).view(np.uint16).T)
    assert np.array_equal(kv.vzero[:, :ctx], lo[..., 0].astype(np.float16).view(np.uint16).T)
    # K shadow holds every row; complete groups are int4 per channel over 32 tokens, the open group is untouched
    assert np.array_equal(kv.kshadow[:, :ctx], k16.transpose(1, 0, 2))
    ng = ctx // 32
    kg = k[:ng * 32].reshape(ng, 32, shape.hkv, shape.hd)
    lo = kg.min(1, keepdims=True); hi = kg.max(1, keepdims=True)
    q, sc = np_quant(kg, lo, hi)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)       # [ng][32][hkv][hd/2]
    assert np.array_equal(kv.kq[:, :ng], packed.transpose(2, 0, 1, 3))
    assert np.array_equal(kv.kscale[:, :ng], sc[:, 0].astype(np.float16).view(np.uint16).transpose(1, 0, 2))
    assert np.array_equal(kv.kzero[:, :ng], lo[:, 0].astype(np.float16).view(np.uint16).transpose(1, 0, 2))
    assert not kv.kq[:, ng:].any() and not kv.kscale[:, ng:].any()


def test_codec_edge_cases(oracle):
    shape = synth.Shape(2, 1, 64, 0, 1.0)
    kv = oracle.KvCache(1, 64, 64)
    # constant rows: hi == lo -> inv = 0, all codes 0, scale 0, zero = value (src/attention_gqa.cu:149)
    k = np.full((32, 1, 64), np.float16(1.5)).view(np.uint16); v = np.full((32, 1, 64), np.float16(-2.25)).view(np.uint16)
    oracle.append(kv, 0, k, v)
    assert not kv.kq[:, 0].any() and not kv.vq[:, :32].any()
    assert np.all(kv.kscale[:, 0] == 0) and np.all(kv.kzero[:, 0] == np.float16(1.5).view(np.uint16))
    assert np.all(kv.vzero[:, :32] == np.float16(-2.25).view(np.uint16))
    # a pass that does not reach the 32nd token of a group leaves the group unquantised
    oracle.append(kv, 32, k[:31], v[:31])
    assert not kv.kscale[:, 1].any()
    k2 = k[:1].copy(); k2[0, 0, 0] = np.float16(9.0).view(np.uint16)
    oracle.append(kv, 63, k2, v[:1])
    assert kv.kscale[0, 1, 0] == np.float16(7.5 / 15).view(np.uint16) and (kv.kq[0, 1, 31, 0] & 15) == 15
    del shape


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "kv4_kat_*.npz"))))
def test_oracle_reproduces_golden_files(oracle, path):
    z = np.load(path)
    hq, hkv, hd, rd, ctx, M, max_ctx = [int(x) for x in z["meta"]]
    kv = oracle.KvCache(hkv, hd, max_ctx)
    p = 0
    for n in z["passes"]:
        oracle.append(kv, p, z["k16"][p:p + n], z["v16"][p:p + n]); p += int(n)
    for name, arr in kv.arrays().items():
        assert np.array_equal(arr, z[name]), name
    rope = oracle.rope_table(max_ctx, float(z["theta"]), rd)
    assert np.array_equal(rope, z["rope"])
    out = oracle.attention_exact(z["q16"], kv, ctx, rope, hq, rd, 1.0 / np.sqrt(hd))
    assert np.array_equal(out, z["out"])


@pytest.mark.parametrize("shape,ctx,M,S", [(synth.C1, 300, 1, 32), (synth.C2, 257, 4, 7), (synth.C1, 33, 40, 5)])
def test_split_partials_and_merge_agree_with_exact_attention(oracle, shape, ctx, M, S):
    """The reference-literal split-K path (src/attention_gqa.cu:17-134) and the double-precision softmax agree."""
    kv, _, _ = build_oracle_cache(oracle, shape, ctx + M, seed=5, chunk=29)
    q16 = f16_bits(synth.make_q(shape, M, seed=5))
    rope = oracle.rope_table(kv.max_ctx, shape.theta, shape.rd)
    pm, pl, pacc = oracle.attention_partials(q16, kv, ctx, S, rope, shape.hq, shape.rd, shape.qscale)
    o16 = oracle.combine(pm, pl, pacc, shape.g)
    exact = oracle.attention_exact(q16, kv, ctx, rope, shape.hq, shape.rd, shape.qscale)
    assert_close(bits_f16(o16), exact, "literal vs exact", atol=1e-3, rtol=2e-3)
    # merging per-split triples reproduces the same result (the multi-GPU exchange format)
    for r in range(M):
        parts = np.concatenate([pm[r][..., None], pl[r][..., None], pacc[r]], axis=-1)       # [S][hq][hd+2]
        assert_close(oracle.merge_triples(parts), exact[r], "triple merge", atol=1e-4, rtol=1e-4)


def test_own_group_is_read_from_the_fp16_shadow(oracle):
    """A row inside group g sees keys of g un-quantised even when g is already complete (src/attention_gqa.cu:38-43)."""
    shape = synth.Shape(2, 1, 64, 0, 1.0)
    kv, _, _ = build_oracle_cache(oracle, shape, 64, seed=3)
    q16 = f16_bits(synth.make_q(shape, 1, seed=3))
    base = oracle.attention_exact(q16, kv, 63, None, shape.hq, 0, shape.qscale)          # row at 63: own group 1 from shadow
    kv.kq[:, 1] ^= 0xFF                                                                  # corrupt the int4 copy of group 1
    assert np.array_equal(base, oracle.attention_exact(q16, kv, 63, None, shape.hq, 0, shape.qscale))
    kv.kq[:, 0] ^= 0xFF                                                                  # group 0 IS read as int4
    assert not np.array_equal(base, oracle.attention_exact(q16, kv, 63, None, shape.hq, 0, shape.qscale))


def test_tolerance_constants():
    assert (ATOL, RTOL) == (2e-3, 1e-2)


def test_projection_input_transform_properties(oracle):
    """ysko_xform_a8: a unit vector becomes a row of +-1/sqrt(512) whose codes are all +-127; the transform is its own inverse."""
    n = 1024
    x = np.zeros((1, n), np.float32); x[0, 3] = 1.0; x[0, 512 + 100] = -2.0
    signs = np.ones(n, np.int8); signs[3] = -1
    qx, alpha = oracle.xform_a8(oracle.f32_to_f16_bits(x), signs)
    assert set(np.abs(qx[0, :512]).tolist()) == {127} and set(np.abs(qx[0, 512:]).tolist()) == {127}
    want0 = np.float32(np.float16(np.float32(1.0) * np.float32(0.044194173824159216))) / np.float32(127)
    assert alpha[0, 0] == want0 and alpha[0, 1] == np.float32(np.float16(np.float32(2.0) * np.float32(0.044194173824159216))) / np.float32(127)
    assert qx[0, 0] == -127                                  # H[0][3] = +1, times the flipped sign
