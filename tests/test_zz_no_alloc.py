"""The allocation-free decode entry (yskn_kv4_decode_noalloc) against the regular attention + merge entries.

Collected last on purpose: a run that stops at the first failure has then already exercised everything else."""
import numpy as np
import pytest
import torch

from tests.helpers import gpu_append_all
from yasakani_b200 import synth

pytestmark = pytest.mark.gpu


def test_noalloc_decode_equals_regular_entries_twice_in_a_row():
    from yasakani_b200 import kv4, Kv4Error
    shape, ctx, splits = synth.C2, 5000, 37
    k, v = synth.make_kv(shape, ctx + 2, seed=61)
    layer = kv4.KvLayer(shape.hkv, shape.hd, 5120)
    gpu_append_all(kv4, layer, k, v, [ctx + 2])
    rope = torch.empty((5120, shape.rd // 2, 2), dtype=torch.float32, device="cuda")
    kv4.launch_rope_table_g(rope, 5120, shape.theta, shape.rd)
    for call, pos in enumerate((ctx, ctx + 1)):                  # two calls in a row, different query and position
        q = synth.make_q(shape, 1, seed=61 + call).cuda()
        d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        pm, pl, pacc = kv4.attn_scratch(1, splits, shape.hq, shape.hd)
        want = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
        kv4.launch_attention_gqa(q, layer, 1, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd)
        kv4.launch_attn_combine_gqa(pm, pl, pacc, splits, 1, want, shape.hq, shape.g)
        got = torch.full_like(want, float("nan"))
        kv4.decode_noalloc(q, layer, d_pos, splits, rope, shape.hq, shape.qscale, shape.rd, got)
        torch.cuda.synchronize()
        assert kv4.device_status() == 0
        # same kernels, same inputs, scratch in another place: identical bits
        assert np.array_equal(got.cpu().view(torch.int16).numpy(), want.cpu().view(torch.int16).numpy()), f"call {call}"
    # a request beyond the built-in scratch is refused, not truncated
    with pytest.raises(Kv4Error, match="exceeds the built-in scratch"):
        kv4.decode_noalloc(q, layer, d_pos, 100, rope, shape.hq, shape.qscale, shape.rd, got)


@pytest.mark.parametrize("shape,splits", [
    (synth.Shape(hq=3, hkv=1, hd=128, rd=128, theta=1e6), 5),      # splits * nh = 15: the O plane of the scratch would start 8-byte aligned unpadded
    (synth.Shape(hq=8, hkv=2, hd=64, rd=64, theta=1e6), 6),        # head_dim 64: the CUDA-core kernel, not the tensor-core one
])
def test_noalloc_decode_other_shapes_equal_the_regular_entries(shape, splits):
    from yasakani_b200 import kv4
    ctx = 700
    k, v = synth.make_kv(shape, ctx + 1, seed=62)
    layer = kv4.KvLayer(shape.hkv, shape.hd, 768)
    gpu_append_all(kv4, layer, k, v, [ctx + 1])
    rope = torch.empty((768, shape.rd // 2, 2), dtype=torch.float32, device="cuda")
    kv4.launch_rope_table_g(rope, 768, shape.theta, shape.rd)
    q = synth.make_q(shape, 1, seed=62).cuda()
    d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
    pm, pl, pacc = kv4.attn_scratch(1, splits, shape.hq, shape.hd)
    want = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    kv4.launch_attention_gqa(q, layer, 1, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd)
    kv4.launch_attn_combine_gqa(pm, pl, pacc, splits, 1, want, shape.hq, shape.g)
    for _ in range(2):
        got = torch.full_like(want, float("nan"))
        kv4.decode_noalloc(q, layer, d_pos, splits, rope, shape.hq, shape.qscale, shape.rd, got)
        torch.cuda.synchronize()
        assert kv4.device_status() == 0
        assert np.array_equal(got.cpu().view(torch.int16).numpy(), want.cpu().view(torch.int16).numpy())


def test_noalloc_decode_rejects_what_its_sibling_entries_reject():
    """Bad arguments come back as -1 with a message before anything is enqueued, never as a device fault."""
    import ctypes as C
    from yasakani_b200 import _lib, kv4
    shape = synth.C2
    layer = kv4.KvLayer(shape.hkv, shape.hd, 128)
    rope = torch.zeros((128, shape.rd // 2, 2), dtype=torch.float32, device="cuda")
    q = torch.zeros((1, shape.hq, shape.hd), dtype=torch.float16, device="cuda")
    o16 = torch.zeros_like(q)
    d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    L = _lib.load()

    def call(s, act_dtype=_lib.F16, rope_ptr=rope.data_ptr(), g_hq=shape.hq):
        return L.yskn_kv4_decode_noalloc(q.data_ptr(), C.byref(s), 128, d_pos.data_ptr(), 4, rope_ptr, shape.hkv, g_hq, shape.hd, shape.rd,
                                         C.c_float(shape.qscale), act_dtype, o16.data_ptr(), None)

    s = layer.struct(); s.vzero = None
    assert call(s) == -1 and b"null cache array" in L.yskn_kv4_last_error()
    assert call(layer.struct(), act_dtype=_lib.F32) == -1 and b"act_dtype" in L.yskn_kv4_last_error()
    assert call(layer.struct(), rope_ptr=None) == -1 and b"rope" in L.yskn_kv4_last_error()
    assert call(layer.struct(), g_hq=shape.hkv * 9) == -1                          # more than 8 query heads per kv-head
    torch.cuda.synchronize()
    assert kv4.device_status() == 0
