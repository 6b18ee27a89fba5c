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
