"""GPU parity of the KV4 codec through the C ABI: packed cache bit-exact against the CPU oracle."""
import glob
import os

import numpy as np
import pytest
import torch

from tests.helpers import build_oracle_cache, f16_bits, gpu_append_all
from yasakani_b200 import synth

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _compare(layer, okv):
    got = layer.to_numpy()
    for name, want in okv.arrays().items():
        assert np.array_equal(got[name].reshape(want.shape), want), f"{name} differs"


@pytest.mark.parametrize("shape,ctx,passes", [
    (synth.C1, 200, [1] * 40 + [31, 33, 64, 32]),               # single-token decode appends, then ragged chunks
    (synth.C2, 291, [97, 1, 1, 30, 2, 160]),
    (synth.C2, 100, [30] + [1] * 70),                           # one-row passes that close groups 0, 1 and 2 inside the append launch
    (synth.Shape(4, 1, 64, 64, 1e4), 70, [1] * 70),
    (synth.Shape(4, 1, 64, 64, 1e4), 96, [96]),
    (synth.C2, 8192, [8192]),                                   # one prefill-sized pass (C5's prompt length)
])
def test_append_is_bit_exact(oracle, shape, ctx, passes):
    from yasakani_b200 import kv4
    assert sum(passes) == ctx
    k, v = synth.make_kv(shape, ctx, seed=21)
    okv = oracle.KvCache(shape.hkv, shape.hd, ((ctx + 127) // 64) * 64)
    k16, v16 = f16_bits(k), f16_bits(v)
    p = 0
    for n in passes:
        oracle.append(okv, p, k16[p:p + n], v16[p:p + n]); p += n
    layer = kv4.KvLayer(shape.hkv, shape.hd, okv.max_ctx)
    gpu_append_all(kv4, layer, k, v, passes)
    _compare(layer, okv)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_append_converts_bf16_and_f32_rows_like_the_oracle(oracle, dtype):
    from yasakani_b200 import kv4
    shape, ctx = synth.C2, 96
    k, v = synth.make_kv(shape, ctx, seed=22, dtype=torch.bfloat16)
    if dtype == torch.float32:                                  # values that do not fit fp16 exactly
        k, v = k.float() * 1.0003, v.float() * 0.9997
    okv = oracle.KvCache(shape.hkv, shape.hd, 128)
    oracle.append(okv, 0, f16_bits(k.to(torch.float16)), f16_bits(v.to(torch.float16)))      # RNE to fp16 first
    layer = kv4.KvLayer(shape.hkv, shape.hd, 128)
    gpu_append_all(kv4, layer, k, v, [ctx])
    _compare(layer, okv)


def test_edge_rows_constant_and_extreme(oracle):
    from yasakani_b200 import kv4
    shape = synth.Shape(8, 2, 128, 0, 1.0)
    k, v = synth.make_kv(shape, 64, seed=23)
    k[0:32, 0] = 1.5; v[3] = -2.25                               # hi == lo: scale 0, codes 0
    k[40, 1, 5] = 60000.0; v[41, 0, 7] = -60000.0                # near the fp16 limit
    k[50, 0, 9] = 6e-8; v[51, 1, 11] = 6e-8                      # fp16 subnormal
    okv = oracle.KvCache(shape.hkv, shape.hd, 64)
    oracle.append(okv, 0, f16_bits(k), f16_bits(v))
    layer = kv4.KvLayer(shape.hkv, shape.hd, 64)
    gpu_append_all(kv4, layer, k, v, [64])
    _compare(layer, okv)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLD, "kv4_kat_*.npz"))))
def test_append_reproduces_golden_cache(path):
    from yasakani_b200 import kv4
    z = np.load(path)
    hq, hkv, hd, rd, ctx, M, max_ctx = [int(x) for x in z["meta"]]
    layer = kv4.KvLayer(hkv, hd, max_ctx)
    k = torch.from_numpy(z["k16"].view(np.int16)).view(torch.float16); v = torch.from_numpy(z["v16"].view(np.int16)).view(torch.float16)
    gpu_append_all(kv4, layer, k, v, [int(n) for n in z["passes"]])
    got = layer.to_numpy()
    for name in ("kq", "kscale", "kzero", "kshadow", "vq", "vscale", "vzero"):
        assert np.array_equal(got[name].reshape(z[name].shape), z[name]), name


def test_group_quant_entry_alone_and_idempotent(oracle):
    """Writing shadow rows and calling only the group-quant entry gives the same groups; a second call changes nothing."""
    from yasakani_b200 import kv4
    shape, ctx = synth.C2, 128
    okv, k16, v16 = build_oracle_cache(oracle, shape, ctx, seed=24, max_ctx=128)
    layer = kv4.KvLayer(shape.hkv, shape.hd, 128)
    layer.kshadow.copy_(torch.from_numpy(okv.kshadow.view(np.int16)).view(torch.float16))
    d_pos = torch.tensor([0], dtype=torch.int32, device="cuda")
    for _ in range(2):
        kv4.launch_kv_group_quant_g(layer, d_pos, ctx)
        torch.cuda.synchronize()
        got = layer.to_numpy()
        for name in ("kq", "kscale", "kzero"):
            assert np.array_equal(got[name].reshape(getattr(okv, name).shape), getattr(okv, name)), name


def test_rope_table_matches_oracle(oracle):
    from yasakani_b200 import kv4
    for max_ctx, theta, rd in [(4096, 1e6, 128), (8192, 1e7, 64)]:
        out = torch.empty((max_ctx, rd // 2, 2), dtype=torch.float32, device="cuda")
        kv4.launch_rope_table_g(out, max_ctx, theta, rd)
        torch.cuda.synchronize()
        want = oracle.rope_table(max_ctx, theta, rd)
        got = out.cpu().numpy()
        # identical angle (fp32 product), double-precision cos/sin rounded once: equal up to one fp32 ulp
        assert np.max(np.abs(got - want)) <= 1.2e-7
        assert np.mean(got == want) > 0.99


def test_bad_arguments_are_rejected_with_a_message():
    from yasakani_b200 import kv4, Kv4Error
    layer = kv4.KvLayer(2, 128, 64)
    d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    rows = torch.zeros((1, 2, 128), dtype=torch.float16, device="cuda")
    layer.hd = 96                                                 # unsupported head_dim
    with pytest.raises(Kv4Error, match="unsupported head_dim"):
        kv4.launch_kv_append(layer, rows[:, :, :96].contiguous(), rows[:, :, :96].contiguous(), d_pos, 1)


def test_projection_input_transform_is_bit_exact(oracle):
    """yskn_kv4_xform_a8 (sign flip, Hadamard-512, int8 + scale per 512 values) against the oracle, on rows that include
    an all-zero group (scale 0) and large values."""
    from yasakani_b200 import kv4
    M, n = 5, 24 * 256
    g = torch.Generator().manual_seed(77)
    rows = (torch.randn((M, n), generator=g) * torch.exp(torch.randn((M, 1), generator=g))).to(torch.float16)
    rows[2, 512:1024] = 0
    rows[3, :512] = 60000.0
    signs = (torch.randint(0, 2, (n,), generator=g) * 2 - 1).to(torch.int8)
    qx = torch.empty((M, n), dtype=torch.int8, device="cuda"); alpha = torch.empty((M, n // 512), dtype=torch.float32, device="cuda")
    kv4.launch_xform_a8(rows.cuda().view(M, 24, 256), signs.cuda(), qx, alpha)
    torch.cuda.synchronize()
    want_q, want_a = oracle.xform_a8(f16_bits(rows), signs.numpy())
    assert np.array_equal(qx.cpu().numpy(), want_q)
    assert np.array_equal(alpha.cpu().numpy().view(np.uint32), want_a.view(np.uint32))
    assert float(alpha[2, 1]) == 0.0 and not qx[2, 512:1024].any()


def test_copy_kernel_moves_small_buffers_between_pinned_host_memory_and_the_device():
    """yskn_kv4_copy: host -> device -> host by kernels, also as nodes of a captured graph that is replayed after the host
    buffer changed (host memory is read past the caches); misaligned sizes are rejected."""
    from yasakani_b200 import kv4, Kv4Error
    h = torch.randn(8192, generator=torch.Generator().manual_seed(9)).half().pin_memory()
    d = torch.empty(8192, dtype=torch.float16, device="cuda")
    back = torch.zeros(8192, dtype=torch.float16).pin_memory()
    kv4.copy_small(d, h); kv4.copy_small(back, d)
    torch.cuda.synchronize()
    assert torch.equal(back, h) and torch.equal(d.cpu(), h)
    g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            kv4.copy_small(d, h); kv4.copy_small(back, d)
    for i in range(3):
        h.fill_(float(i + 1))
        g.replay(); torch.cuda.synchronize()
        assert float(back[5]) == i + 1 and float(back[-1]) == i + 1
    with pytest.raises(Kv4Error, match="multiples of 16"):
        kv4.copy_small(d[:3], h[:3])
    with pytest.raises(ValueError, match="pinned"):
        kv4.copy_small(d, torch.zeros(8192, dtype=torch.float16))
