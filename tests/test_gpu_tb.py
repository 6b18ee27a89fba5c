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
