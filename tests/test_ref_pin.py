"""Pins the CPU oracle (and our kernels) against the reference's own CUDA kernels.

oracle/_ref/libyskn_ref_kv4.so is compiled from the reference's source files where they lie
(oracle/Makefile, target `ref`) and travels to the GPU box as a built file.  It covers the K group codec
(kv_group_quant_g_kernel), the generic GQA decode kernel and its merge kernel, and the per-token V codec inside
the reference's fused QKV epilogue (qkv_post_kernel, src/post_kernels.cu:26-82), driven so that its K branch
stores the very fp16 row its V branch quantises.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from tests.helpers import assert_close, bits_f16, build_oracle_cache, f16_bits, gpu_attention
from yasakani_b200 import synth

pytestmark = pytest.mark.gpu
REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libyskn_ref_kv4.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref not built (reference tree was not mounted at build time)")
    return C.CDLL(REF)


def _ptrs(layer):
    return [C.c_void_p(t.data_ptr()) for t in layer.tensors()]


@pytest.mark.parametrize("shape", [synth.C2, synth.C1])
def test_oracle_group_codec_equals_reference_kernel_bit_for_bit(oracle, ref, shape):
    from yasakani_b200 import kv4
    ctx = 160
    okv, k16, v16 = build_oracle_cache(oracle, shape, ctx, seed=41, max_ctx=192)
    ours = kv4.KvLayer(shape.hkv, shape.hd, 192)
    ours.kshadow.copy_(torch.from_numpy(okv.kshadow.view(np.int16)).view(torch.float16))
    d_pos = torch.tensor([0], dtype=torch.int32, device="cuda")
    rc = ref.yref_kv_group_quant_g(*_ptrs(ours), C.c_void_p(d_pos.data_ptr()), ctx, 192, shape.hkv, shape.hd, None)
    assert rc == 0
    torch.cuda.synchronize()
    got = ours.to_numpy()
    for name in ("kq", "kscale", "kzero"):
        assert np.array_equal(got[name].reshape(getattr(okv, name).shape), getattr(okv, name)), name


def test_v_codec_equals_reference_qkv_epilogue_bit_for_bit(oracle, ref):
    """The reference's V branch (src/post_kernels.cu:64-82) exists for hd 128 / 4 kv-heads only.  With one GEMV slice,
    tau = 1, no bias and the same `part` and sign vector for K and V, block 7 stores round_f16(inv_h512(part)) into
    kshadow and block 8 quantises the identical fp16 row into vq / vscale / vzero: kshadow is the witness of the V
    codec's input.  The oracle's and the library's V codec over those shadow rows must reproduce the reference's bytes."""
    from yasakani_b200 import kv4
    hkv, hd, M, max_ctx, pos0 = 4, 128, 77, 192, 23
    g = torch.Generator().manual_seed(4242)
    part = torch.randn((M, 512), generator=g) * torch.exp(torch.rand((1, 512), generator=g) * 3.0 - 1.5)
    part[5, 128:256] = 0.25                                        # a constant row: hi == lo, scale 0 (src/post_kernels.cu:76)
    part[6] = 0.0
    signs = (torch.randint(0, 2, (512,), generator=g) * 2 - 1).to(torch.int8)
    dev = "cuda"
    d = dict(part=part.to(dev), ones=torch.ones(512, device=dev), signs=signs.to(dev), zb=torch.zeros(512, dtype=torch.float16, device=dev),
             qpart=torch.zeros((M, 3584), device=dev), qtau=torch.ones(3584, device=dev), qsigns=torch.ones(3584, dtype=torch.int8, device=dev),
             qbias=torch.zeros(3584, dtype=torch.float16, device=dev), q16=torch.zeros((M, 28, 128), dtype=torch.float16, device=dev))
    theirs = kv4.KvLayer(hkv, hd, max_ctx)
    d_pos = torch.tensor([pos0], dtype=torch.int32, device=dev)
    P = lambda t: C.c_void_p(t.data_ptr())
    rc = ref.yref_qkv_post_kv(P(d["part"]), P(d["ones"]), P(d["signs"]), P(d["zb"]), P(d["qpart"]), P(d["qtau"]), P(d["qsigns"]), P(d["qbias"]),
                              P(d["q16"]), *_ptrs(theirs), P(d_pos), M, max_ctx, None)
    assert rc == 0
    torch.cuda.synchronize()
    got = theirs.to_numpy()
    shadow = got["kshadow"].reshape(hkv, max_ctx, hd)[:, pos0:pos0 + M]            # [hkv][M][hd] fp16 bits: the rows both branches saw
    rows = np.ascontiguousarray(shadow.transpose(1, 0, 2))                         # [M][hkv][hd]
    # The K branch adds a +0.0 bias before it stores, which turns -0.0 into +0.0; the V branch has no bias.  For the all-zero
    # input row the V branch therefore saw 0 * sign = -0.0 wherever the sign is -1: restore those signs in the witness.
    neg = (signs.numpy().reshape(hkv, hd) < 0)
    assert (rows[6] == 0).all()
    rows[6] = np.where(neg, 0x8000, 0).astype(np.uint16)
    assert len(np.unique(rows)) > 1000                                             # the epilogue really ran on the random rows
    # oracle: the V codec over the witnessed rows
    okv = oracle.KvCache(hkv, hd, max_ctx)
    oracle.append(okv, pos0, rows, rows)
    for name in ("vq", "vscale", "vzero"):
        want = getattr(okv, name)[:, pos0:pos0 + M]
        have = got[name].reshape(getattr(okv, name).shape)[:, pos0:pos0 + M]
        assert np.array_equal(have, want), f"oracle V codec differs from the reference's qkv_post_kernel in {name}"
    # the library's codec over the same rows
    ours = kv4.KvLayer(hkv, hd, max_ctx)
    r16 = torch.from_numpy(rows.view(np.int16)).view(torch.float16).cuda()
    kv4.launch_kv_append(ours, r16, r16, d_pos, M)
    torch.cuda.synchronize()
    mine = ours.to_numpy()
    for name in ("vq", "vscale", "vzero", "kshadow"):
        a = mine[name].reshape(getattr(okv, name).shape)[:, pos0:pos0 + M]
        b = got[name].reshape(getattr(okv, name).shape)[:, pos0:pos0 + M]
        if name == "kshadow":                                                      # the library stores the row as given; the reference's K branch turned -0.0 into +0.0
            a = np.where(a == 0x8000, 0, a); b = np.where(b == 0x8000, 0, b)
        assert np.array_equal(a, b), f"library V codec differs from the reference's qkv_post_kernel in {name}"


@pytest.mark.parametrize("shape,ctx,M", [(synth.C2, 2100, 1), (synth.C2, 700, 3), (synth.Shape(28, 4, 128, 128, 1e6), 1500, 2)])
def test_reference_attention_kernel_agrees_with_oracle_and_with_ours(oracle, ref, shape, ctx, M):
    from yasakani_b200 import kv4
    S = 32
    okv, _, _ = build_oracle_cache(oracle, shape, ctx + M, seed=42, chunk=50)
    layer = kv4.KvLayer(shape.hkv, shape.hd, okv.max_ctx).load_numpy(okv.arrays())
    q = synth.make_q(shape, M, seed=42)
    rope_np = oracle.rope_table(okv.max_ctx, shape.theta, shape.rd)
    rope = torch.from_numpy(rope_np).cuda()
    dq = q.cuda(); d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(M, S, shape.hq, shape.hd)
    rc = ref.yref_attention_gqa(C.c_void_p(dq.data_ptr()), *_ptrs(layer), okv.max_ctx, M, C.c_void_p(d_pos.data_ptr()), S,
                                C.c_void_p(pm.data_ptr()), C.c_void_p(pl.data_ptr()), C.c_void_p(pacc.data_ptr()),
                                C.c_void_p(rope.data_ptr()), shape.hkv, shape.hq, C.c_float(shape.qscale), shape.g, shape.hd, shape.rd, None)
    assert rc == 0
    n = shape.hq * shape.hd
    signs = (torch.randint(0, 2, (n,), generator=torch.Generator().manual_seed(9)) * 2 - 1).to(torch.int8).cuda()
    qx = torch.empty((M, n), dtype=torch.int8, device="cuda")
    alpha = torch.empty((M, n // 512), dtype=torch.float32, device="cuda")
    o_ref = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    rc = ref.yref_attn_combine_gqa_xform(C.c_void_p(pm.data_ptr()), C.c_void_p(pl.data_ptr()), C.c_void_p(pacc.data_ptr()), S, M, None,
                                         C.c_void_p(o_ref.data_ptr()), None, shape.hq, shape.g, shape.hd, C.c_void_p(signs.data_ptr()),
                                         C.c_void_p(qx.data_ptr()), C.c_void_p(alpha.data_ptr()), None)
    assert rc == 0
    torch.cuda.synchronize()
    # (0) the int8 input of the next projection: the library's and the oracle's transform of the reference's own o16 rows
    #     reproduce the reference kernel's codes and scales bit for bit (src/attention_gqa.cu:135-139, src/a8_prologue.cuh:122-133)
    qx2 = torch.empty_like(qx); alpha2 = torch.empty_like(alpha)
    kv4.launch_xform_a8(o_ref, signs, qx2, alpha2)
    torch.cuda.synchronize()
    assert torch.equal(qx2, qx) and torch.equal(alpha2.view(torch.int32), alpha.view(torch.int32)), "library transform differs from the reference's"
    oqx, oal = oracle.xform_a8(f16_bits(o_ref.cpu()).reshape(M, n), signs.cpu().numpy())
    assert np.array_equal(oqx, qx.cpu().numpy()) and np.array_equal(oal.view(np.uint32), alpha.cpu().numpy().view(np.uint32)), "oracle transform differs"
    o_ref = o_ref.float().cpu().numpy()
    # (1) the reference's partials against the oracle's literal restatement of the same kernel
    opm, opl, opacc = oracle.attention_partials(f16_bits(q), okv, ctx, S, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(pm.cpu().numpy(), opm, "pm", atol=1e-4, rtol=1e-5)
    assert_close(pl.cpu().numpy(), opl, "pl", atol=1e-4, rtol=1e-4)
    assert_close(pacc.cpu().numpy(), opacc, "pacc", atol=1e-3, rtol=1e-3)
    # (2) the reference's final output against the tolerance oracle, and (3) against our kernels
    exact = oracle.attention_exact(f16_bits(q), okv, ctx, rope_np, shape.hq, shape.rd, shape.qscale)
    assert_close(o_ref, exact, "reference vs exact oracle", atol=1e-3, rtol=2e-3)
    ours, _ = gpu_attention(kv4, layer, q, ctx, S, rope, shape)
    assert_close(ours, o_ref, "ours vs reference kernels")


def test_rotate_int8_row_codec_equals_the_reference_probe_bit_for_bit(oracle):
    """Family-B row codec, step 1: the reference's own probe (yskn_kvx_probe, src/kvx_probe.cu:22-36, compiled from its
    source into oracle/_ref/libyskn_ref_kvx.so) against the CPU oracle and against this library's probe."""
    from yasakani_b200 import kvx
    path = os.path.join(os.path.dirname(REF), "libyskn_ref_kvx.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (reference tree was not mounted at build time)")
    ref = C.CDLL(path)
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((256, 256)) * np.exp(rng.uniform(np.log(0.05), np.log(20.0), (256, 1)))).astype(np.float32)
    x[5] = 0.0
    q = np.empty((256, 256), dtype=np.int8); sc = np.empty(256, dtype=np.float32); y = np.empty_like(x)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    assert ref.yskn_kvx_codec() in (2, 3)              # rotation + INT8 branches (src/kvx_codec.cuh:11-15)
    assert ref.yskn_kvx_probe(p(x), p(q), p(sc), p(y), 256) == 0
    oq, osc = oracle.kvx_encode(x)
    assert np.array_equal(q, oq)
    assert np.array_equal(sc.view(np.uint32), osc.view(np.uint32))
    assert np.array_equal(y.view(np.uint32), oracle.kvx_decode(oq, osc).view(np.uint32))
    gq, gsc, gy = kvx.probe(x)
    assert np.array_equal(gq, q) and np.array_equal(gsc.view(np.uint32), sc.view(np.uint32)) and np.array_equal(gy.view(np.uint32), y.view(np.uint32))


@pytest.mark.parametrize("ctx,M", [(3000, 1), (700, 3)])
def test_int8_row_decode_agrees_with_the_reference_kernel_and_the_oracle(oracle, ctx, M):
    """Family-B decode over INT8 rows: the reference's q35_attention_kernel<KV8> (src/q35_kernels.cu:1176-1281, compiled
    from its source into oracle/_ref/libyskn_ref_q35.so) against the exact oracle and against this library's kernel,
    each merged by yskn_kv8_combine without the rotation."""
    from yasakani_b200 import kvx
    path = os.path.join(os.path.dirname(REF), "libyskn_ref_q35.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (reference tree was not mounted at build time)")
    ref = C.CDLL(path)
    nh, kvh, hd = C.c_int(), C.c_int(), C.c_int()
    ref.yref_q35_shape(C.byref(nh), C.byref(kvh), C.byref(hd))
    nh, kvh = nh.value, kvh.value
    assert hd.value == 256
    rng = np.random.default_rng(ctx)
    n = ctx + M
    max_ctx = ((n + 63) // 64) * 64
    k8 = np.zeros((kvh, max_ctx, 256), np.int8); v8 = np.zeros_like(k8)
    ks = np.zeros((kvh, max_ctx), np.float32); vs = np.zeros_like(ks)
    for h in range(kvh):
        k8[h, :n], ks[h, :n] = oracle.kvx_encode(rng.standard_normal((n, 256)).astype(np.float32) * 1.5)
        v8[h, :n], vs[h, :n] = oracle.kvx_encode(rng.standard_normal((n, 256)).astype(np.float32))
    q = torch.from_numpy(oracle.kvx_rotate(rng.standard_normal((M * nh, 256)).astype(np.float32)).reshape(M, nh, 256)).to(torch.bfloat16).cuda()
    d = [torch.from_numpy(a).cuda() for a in (k8, v8, ks, vs)]
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    S = 32
    want = oracle.kv8_attention_exact(q.float().cpu().numpy(), k8, v8, ks, vs, ctx)

    def merged(pm, pl, pacc):
        o = torch.empty((M, nh, 256), dtype=torch.float16, device="cuda")
        kvx.launch_kv8_combine(pm, pl, pacc, S, M, nh, o, inverse_rotate=False)
        torch.cuda.synchronize()
        return o.float().cpu().numpy()

    pm = torch.empty((M, S, nh), device="cuda"); pl = torch.empty_like(pm); pacc = torch.empty((M, S, nh, 256), device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    assert ref.yref_q35_attention_kv8(p(q), p(d[0]), p(d[1]), p(d[2]), p(d[3]), max_ctx, M, p(d_pos), S, p(pm), p(pl), p(pacc), None) == 0
    torch.cuda.synchronize()
    theirs = merged(pm, pl, pacc)
    assert_close(theirs, want, "reference INT8-row kernel vs exact oracle")
    pm2 = torch.empty_like(pm); pl2 = torch.empty_like(pl); pacc2 = torch.empty_like(pacc)
    kvx.launch_kv8_attention(q, *d, M, d_pos, S, pm2, pl2, pacc2, nh)
    ours = merged(pm2, pl2, pacc2)
    assert_close(ours, want, "this library's INT8-row kernel vs exact oracle")
    assert_close(ours, theirs, "this library's INT8-row kernel vs the reference kernel")


# ---------------------------------------------------------------------------------------------------------------
# Family B, step 2: the trellis ("CDQ") re-quantisation and its payload against the reference's own probes
# (src/kvx_probe.cu built with YSKN_KVX_MODE=3: yskn_tb_probe = tb_fakequant, yskn_tbp_pack_unpack = the fast encoder
# with its packer), on the synthetic profile blob.
REF_TB = os.path.join(os.path.dirname(REF), "libyskn_ref_tb.so")


def test_trellis_oracle_and_encoder_equal_the_reference_probes_bit_for_bit(oracle):
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    from make_kvqp_blob import make_blob
    from yasakani_b200 import kvx
    if not os.path.exists(REF_TB):
        pytest.skip("oracle/_ref/libyskn_ref_tb.so not built (reference tree was not mounted at build time)")
    R = C.CDLL(REF_TB)
    blob = make_blob(nm=5)
    rows = 128
    rng = np.random.default_rng(77)
    x = (rng.standard_normal((rows, 256)) * np.exp(0.5 * rng.standard_normal((rows, 1)))).astype(np.float32)
    grp = np.arange(rows, dtype=np.int32)                                  # every group record once
    pos = rng.integers(0, 300, rows).astype(np.int32); pos[::9] = 2        # some rows below their guard position
    want = oracle.tb_encode(blob, x, grp, pos)
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    bb = np.frombuffer(blob, np.uint8)
    # (1) tb_fakequant (src/kvq_gpu.cuh:54-148)
    y1 = np.empty_like(x)
    assert R.yskn_tb_probe(P(bb), C.c_size_t(bb.size), P(x), P(grp), P(pos), P(y1), rows) == 0
    assert np.array_equal(y1.view(np.uint32), want["y"].view(np.uint32)), "oracle differs from the reference's tb_fakequant"
    # (2) the fast encoder, its MSB-first packer and side words (src/kvq_fast.cuh:113-232), and the reference's own unpack
    stride = 160
    y2 = np.empty_like(x); ydec = np.empty_like(x)
    pay = np.zeros((rows, stride), np.uint8); side = np.zeros((rows, 2), np.uint32); ms = np.zeros(2, np.float32)
    assert R.yskn_tbp_pack_unpack(P(bb), C.c_size_t(bb.size), P(x), P(grp), P(pos), rows, stride, P(y2), P(pay), P(side), P(ydec), P(ms)) == 0
    packed = want["kb"] > 0
    assert np.array_equal(y2.view(np.uint32), want["y"].view(np.uint32)), "oracle differs from the reference's fast encoder"
    assert np.array_equal(pay.view(np.uint32).reshape(rows, 40)[packed], want["pay"][packed]), "payload"
    assert np.array_equal(side[packed], want["side"][packed]), "side words"
    assert np.array_equal(oracle.tb_unpack(blob, grp, pos, want["pay"], want["side"], x).view(np.uint32), ydec.view(np.uint32)), "oracle unpack differs from the reference's"
    # (3) the library's encoder on the same rows
    y3, pay3, side3 = kvx.tb_encode(kvx.TrellisProfile(blob), torch.from_numpy(x).cuda(), torch.from_numpy(grp).cuda(), torch.from_numpy(pos).cuda(), pay_stride=stride)
    torch.cuda.synchronize()
    assert np.array_equal(y3.cpu().numpy().view(np.uint32), y2.view(np.uint32))
    assert np.array_equal(pay3.cpu().numpy()[packed], pay[packed]) and np.array_equal(side3.cpu().numpy().view(np.uint32)[packed], side[packed])
    back = kvx.tb_decode(kvx.TrellisProfile(blob), pay3, side3, torch.from_numpy(grp).cuda(), torch.from_numpy(pos).cuda(), yin=torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy().view(np.uint32), ydec.view(np.uint32)), "library unpack differs from the reference's tba_unpack_kernel"


@pytest.mark.parametrize("pm", [1, 0], ids=["portable-math", "default-math"])
def test_attn_post_equals_the_reference_kernel_bit_for_bit(oracle, pm):
    """The reference's q35_attn_post_kernel (src/q35_kernels.cu:1013-1065, compiled from its source) against this library's
    yskn_kvx_attn_post and, in the portable-math mode, the CPU oracle.  The reference kernel starts from GEMV partial sums:
    it is driven with one slice, tau = 1, signs = +1 and partial sums whose upper 256 entries per block are zero, which makes
    the two halves of a block's 512 projection values equal.  The gate half, which the kernel stores untouched (gate16), is
    then the witness of the values its query half normalises; key and value blocks get the partial sums of query heads
    0 / 1, so their two heads see the same witnessed rows."""
    from yasakani_b200 import kvx
    path = os.path.join(os.path.dirname(REF), "libyskn_ref_q35.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref not built (reference tree was not mounted at build time)")
    ref = C.CDLL(path)
    nh, kvh, hd = C.c_int(), C.c_int(), C.c_int()
    ref.yref_q35_shape(C.byref(nh), C.byref(kvh), C.byref(hd))
    nh, kvh = nh.value, kvh.value
    assert hd.value == 256 and kvh == 4
    M, rd, max_ctx, pos0, eps = 5, 64, 96, 70, 1e-6
    g = torch.Generator().manual_seed(4242)
    part_q = torch.zeros((M, nh, 512))
    part_q[:, :, :256] = torch.randn((M, nh, 256), generator=g) * torch.exp(torch.rand((1, nh, 1), generator=g) * 3.0 - 1.0) * 16.0
    part_q[1, 2] = 0.0                                             # an all-zero head
    part_k = part_q[:, :2].reshape(M, 1024).contiguous()           # key heads (0, 1) <- query head 0, (2, 3) <- query head 1
    part_v = part_k.clone()
    rng = np.random.default_rng(3)
    from tests.helpers import bf16_bits
    qn_w = bf16_bits(rng.standard_normal(256) * 0.2); kn_w = bf16_bits(rng.standard_normal(256) * 0.2 + 0.5)
    rope_np = oracle.rope_table(max_ctx, 1e7, rd)
    dev = "cuda"
    bf = lambda bits: torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(dev)
    t = dict(part_q=part_q.reshape(M, nh * 512).to(dev), part_k=part_k.to(dev), part_v=part_v.to(dev), ones=torch.ones(nh * 512, device=dev),
             signs=torch.ones(nh * 512, dtype=torch.int8, device=dev), qn_w=bf(qn_w), kn_w=bf(kn_w), rope=torch.from_numpy(rope_np).to(dev),
             d_pos=torch.tensor([pos0], dtype=torch.int32, device=dev))

    def caches():
        return (torch.zeros((kvh, max_ctx, 256), dtype=torch.int8, device=dev), torch.zeros((kvh, max_ctx, 256), dtype=torch.int8, device=dev),
                torch.zeros((kvh, max_ctx), device=dev), torch.zeros((kvh, max_ctx), device=dev))
    P = lambda x: C.c_void_p(x.data_ptr())
    rq16 = torch.empty((M, nh, 256), dtype=torch.bfloat16, device=dev); rgate = torch.empty_like(rq16)
    rk8, rv8, rks, rvs = caches()
    ref.yref_q35_attn_post.argtypes = [C.c_void_p] * 7 + [C.c_float, C.c_int] + [C.c_void_p] * 8 + [C.c_int, C.c_int, C.c_void_p]
    rc = ref.yref_q35_attn_post(P(t["part_q"]), P(t["part_k"]), P(t["part_v"]), P(t["ones"]), P(t["signs"]), P(t["qn_w"]), P(t["kn_w"]), eps, M,
                                P(t["d_pos"]), P(t["rope"]), P(rq16), P(rgate), P(rk8), P(rv8), P(rks), P(rvs), max_ctx, pm, None)
    torch.cuda.synchronize()
    assert rc == 0
    # the witnessed projection rows: query head h = [y_h | y_h]; key / value head j = y of query head j // 2
    y = rgate                                                      # bf16 [M][nh][256]
    assert float(y.float().abs().max()) > 0.5
    q_rows = torch.cat([y, y], dim=2).contiguous()
    kv_rows = y[:, [0, 0, 1, 1]].contiguous()
    q16 = torch.empty_like(rq16); gate16 = torch.empty_like(rq16)
    k8, v8, ks, vs = caches()
    kvx.launch_attn_post(q_rows, kv_rows, kv_rows, t["qn_w"], t["kn_w"], eps, t["d_pos"], t["rope"], rd, q16, gate16, k8, ks, v8, vs, pm=bool(pm))
    torch.cuda.synchronize()
    i16 = lambda x: x.view(torch.int16)
    assert torch.equal(i16(q16), i16(rq16)), f"q16 differs in {(i16(q16) != i16(rq16)).sum().item()} elements"
    assert torch.equal(i16(gate16), i16(rgate))
    assert torch.equal(k8, rk8) and torch.equal(v8, rv8)
    assert torch.equal(ks.view(torch.int32), rks.view(torch.int32)) and torch.equal(vs.view(torch.int32), rvs.view(torch.int32))
    assert int((rk8[:, pos0:pos0 + M] != 0).sum()) > 1000 and not rk8[:, :pos0].any()
    if pm:
        bits = lambda x: x.view(torch.int16).cpu().numpy().view(np.uint16)
        ok8 = np.zeros((kvh, max_ctx, 256), np.int8); ov8 = np.zeros_like(ok8)
        oks = np.zeros((kvh, max_ctx), np.float32); ovs = np.zeros_like(oks)
        oq16, _ = oracle.kvx_attn_post(bits(q_rows), bits(kv_rows), bits(kv_rows), qn_w, kn_w, eps, pos0, rope_np, rd, max_ctx, ok8, oks, ov8, ovs)
        assert np.array_equal(oq16, bits(rq16)) and np.array_equal(ok8, rk8.cpu().numpy()) and np.array_equal(ov8, rv8.cpu().numpy())
        assert np.array_equal(oks.view(np.uint32), rks.cpu().numpy().view(np.uint32)) and np.array_equal(ovs.view(np.uint32), rvs.cpu().numpy().view(np.uint32))
