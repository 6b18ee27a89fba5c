"""The trellis ("CDQ") row codec on the GPU: the library's encoder against the CPU oracle, bit for bit, on the synthetic
"KVQP v1" profile blob (the shipping blob lives in the model folder, not in the reference repository)."""
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_kvqp_blob import make_blob  # noqa: E402

pytestmark = pytest.mark.gpu


def _rows(n, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((n, 256)) * np.exp(rng.standard_normal((n, 1)))).astype(np.float32)
    x[3] = 0.0                                                   # rms 0 -> 1, every code 0
    x[5, 10:] = 0.0
    grp = rng.integers(0, 128, n).astype(np.int32)
    grp[:128] = np.arange(128, dtype=np.int32)[:min(n, 128)]     # every group record at least once
    pos = rng.integers(0, 300, n).astype(np.int32)
    pos[::7] = 1                                                 # below the guard position of some groups
    return x, grp, pos


@pytest.mark.parametrize("nm", [5, 9])
def test_encoder_is_bit_exact_with_the_oracle(oracle, nm):
    from yasakani_b200 import kvx
    blob = make_blob(nm=nm)
    x, grp, pos = _rows(200, 31 + nm)
    want = oracle.tb_encode(blob, x, grp, pos)
    prof = kvx.TrellisProfile(blob)
    assert prof.nm == nm
    y, pay, side = kvx.tb_encode(prof, torch.from_numpy(x).cuda(), torch.from_numpy(grp).cuda(), torch.from_numpy(pos).cuda())
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want["y"].view(np.uint32)), "re-quantised rows differ"
    got_pay = pay.cpu().numpy().view(np.uint32).reshape(200, 40)
    packed = want["kb"] > 0
    assert np.array_equal(got_pay[packed], want["pay"][packed]), "payload differs"
    assert not got_pay[~packed].any()                            # rows below the guard position are not packed
    assert np.array_equal(side.cpu().numpy().view(np.uint32)[packed], want["side"][packed]), "side words differ"
    # and back: the packed rows decode, without the search, to the re-quantised rows (rows that were not packed keep the input)
    back = kvx.tb_decode(prof, pay, side, torch.from_numpy(grp).cuda(), torch.from_numpy(pos).cuda(), yin=torch.from_numpy(x).cuda())
    torch.cuda.synchronize()
    want_back = oracle.tb_unpack(blob, grp, pos, want["pay"], want["side"], x)
    assert np.array_equal(back.cpu().numpy().view(np.uint32), want_back.view(np.uint32)), "decode differs from the oracle"
    assert np.array_equal(back.cpu().numpy(), want["y"])         # by value: a flat code of -0 decodes to +0


def test_blob_check_rejects_what_the_reference_loader_rejects():
    import ctypes as C
    from yasakani_b200 import _lib
    L = _lib.load()
    blob = bytearray(make_blob())
    nm = C.c_int(0)
    buf = (C.c_uint8 * len(blob)).from_buffer(blob)
    assert L.yskn_tb_blob_info(buf, len(blob), C.byref(nm)) == 0 and nm.value == 5
    blob[16] = 128                                               # D must be 256 (src/engine35.cpp:52)
    assert L.yskn_tb_blob_info(buf, len(blob), C.byref(nm)) == -1 and b"D 256" in L.yskn_kv4_last_error()
    assert L.yskn_tb_blob_info(buf, len(blob) - 1, C.byref(nm)) == -1


@pytest.mark.parametrize("ctx,M,splits,dtype", [(700, 1, 5, torch.bfloat16), (333, 3, 4, torch.float16), (2, 2, 3, torch.bfloat16)])
def test_attention_over_packed_rows_equals_attention_over_the_unpacked_rows(oracle, ctx, M, splits, dtype):
    """yskn_tb_attention unpacks every key / value row inside the kernel: its merged result against the exact oracle over the
    rows the oracle's unpack gives for the same payload.  The heads' groups mix trellis and flat records, three code widths,
    rank 0 / 1 / 2 corrections and guarded groups (positions 0..3 stay unpacked and come from the plain rows)."""
    from yasakani_b200 import kvx
    blob = make_blob()
    prof = kvx.TrellisProfile(blob)
    kvh, nh, n = 4, 24, ctx + M
    max_ctx = ((n + 63) // 64) * 64
    grp_k = np.array([8, 15, 21, 34], np.int32); grp_v = np.array([3, 31, 16, 45], np.int32)
    rng = np.random.default_rng(ctx)
    xk = np.zeros((kvh, max_ctx, 256), np.float32); xv = np.zeros_like(xk)
    xk[:, :n] = rng.standard_normal((kvh, n, 256)) * np.exp(rng.uniform(np.log(0.5), np.log(2.0), (kvh, 1, 256)))
    xv[:, :n] = rng.standard_normal((kvh, n, 256))
    pos_rows = np.tile(np.arange(max_ctx, dtype=np.int32), kvh)
    dev = "cuda"
    packed = {}
    for name, x, grp in (("k", xk, grp_k), ("v", xv, grp_v)):
        grp_rows = np.repeat(grp, max_ctx).astype(np.int32)
        _, pay, side = kvx.tb_encode(prof, torch.from_numpy(x.reshape(-1, 256)).to(dev), torch.from_numpy(grp_rows).to(dev), torch.from_numpy(pos_rows).to(dev))
        torch.cuda.synchronize()
        rows = oracle.tb_unpack(blob, grp_rows, pos_rows, pay.cpu().numpy().view(np.uint32).reshape(-1, 40), side.cpu().numpy().view(np.uint32), x.reshape(-1, 256))
        packed[name] = (pay.view(kvh, max_ctx, -1), side.view(kvh, max_ctx, 2), rows.reshape(kvh, max_ctx, 256))
    if n > 4:
        assert np.abs(packed["k"][2][:, 4:n] - xk[:, 4:n]).max() > 1e-3              # the rows really went through the codec
    q = (torch.from_numpy(rng.standard_normal((M, nh, 256)).astype(np.float32)) * 0.7).to(dtype)
    want = oracle.rows_attention_exact(q.float().numpy(), packed["k"][2], packed["v"][2], ctx)
    pm = torch.empty((M, splits, nh), device=dev); pl = torch.empty_like(pm); pacc = torch.empty((M, splits, nh, 256), device=dev)
    d_pos = torch.tensor([ctx], dtype=torch.int32, device=dev)
    kvx.launch_tb_attention(prof, q.to(dev), packed["k"][0], packed["k"][1], packed["v"][0], packed["v"][1], torch.from_numpy(grp_k).to(dev),
                            torch.from_numpy(grp_v).to(dev), M, d_pos, splits, pm, pl, pacc, nh,
                            k_plain=torch.from_numpy(xk).to(dev), v_plain=torch.from_numpy(xv).to(dev))
    o16 = torch.empty((M, nh, 256), dtype=dtype, device=dev)
    kvx.launch_kv8_combine(pm, pl, pacc, splits, M, nh, o16, inverse_rotate=False)
    torch.cuda.synchronize()
    got = o16.float().cpu().numpy()
    err = np.abs(got - want)
    assert (err <= 2e-3 + 1e-2 * np.abs(want)).all(), f"max err {err.max():.3e}"
