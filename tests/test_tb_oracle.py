"""The trellis ("CDQ") row codec's CPU oracle (oracle/tb_oracle.c) on the synthetic profile blob: the blob passes the
reference loader's checks, the payload decodes back to the quantised row, and more bits per value give a smaller error.
(The oracle itself is pinned against the reference's probes on a GPU in tests/test_ref_pin.py.)"""
import os
import struct
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_kvqp_blob import make_blob  # noqa: E402


def _rows(n, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((n, 256)) * np.exp(rng.standard_normal((n, 1)))).astype(np.float32)
    grp = rng.integers(0, 128, n).astype(np.int32)
    pos = rng.integers(0, 300, n).astype(np.int32)
    return x, grp, pos


def _group(blob, g):
    go = struct.unpack_from("<I", blob, struct.unpack_from("<I", blob, 40)[0] + 4 * int(g))[0]
    mode, kk, tix, guard, m, mu = blob[go:go + 6]
    return dict(go=go, mode=mode, kk=kk, tix=tix, guard=guard, m=m, mu=mu)


def test_synthetic_blob_passes_the_reference_loader_checks(oracle):
    blob = make_blob()
    assert oracle.tb_check_blob(blob) == 0
    assert oracle.tb_check_blob(blob[:-1]) != 0 and oracle.tb_check_blob(b"KVQX" + blob[4:]) != 0
    committed = os.path.join(os.path.dirname(__file__), "golden", "kvqp_synthetic.bin")
    assert open(committed, "rb").read() == blob                 # the committed file is what the generator makes


def test_payload_decodes_to_the_quantised_row(oracle):
    blob = make_blob()
    x, grp, pos = _rows(64, 5)
    r = oracle.tb_encode(blob, x, grp, pos)
    seen = set()
    for i in range(64):
        G = _group(blob, grp[i])
        if pos[i] < G["guard"]:
            assert r["kb"][i] == 0 and np.array_equal(r["y"][i], x[i]) and not r["pay"][i].any()
            continue
        kb = 4 if G["mode"] == 1 else G["kk"]
        assert r["kb"][i] == kb and not r["pay"][i, 8 * kb:].any()
        xq = oracle.tb_decode_fields(blob, grp[i], r["pay"][i], r["side"][i, :1].view(np.float32)[0])
        # add the low-rank part and the mean back exactly as the encoder does
        c = r["side"][i, 1:2].view(np.uint16)[:2].view(np.float16).astype(np.float32)
        mu_off = G["go"] + 8
        y = xq.copy()
        base = mu_off + (512 if G["mu"] else 0)
        for j in range(G["m"]):
            u = np.frombuffer(blob, np.float16, 256, base + 512 * j).astype(np.float32)
            y = (y + c[j] * u).astype(np.float32)
        if G["mu"]:
            y = (y + np.frombuffer(blob, np.float16, 256, mu_off).astype(np.float32)).astype(np.float32)
        assert np.array_equal(y, r["y"][i]), f"row {i}"        # by value: a flat code of -0 decodes to +0
        seen.add((G["mode"], kb))
    assert {(0, 3), (0, 4), (0, 5), (1, 4)} <= seen


def test_more_bits_per_value_give_a_smaller_error(oracle):
    blob = make_blob()
    rng = np.random.default_rng(9)
    x = rng.standard_normal((60, 256)).astype(np.float32)
    by_kk = {}
    for g in range(128):
        G = _group(blob, g)
        if G["mode"] == 0 and G["guard"] == 0:
            by_kk.setdefault(G["kk"], g)
    err = {}
    for kk, g in by_kk.items():
        r = oracle.tb_encode(blob, x, np.full(60, g, np.int32), np.full(60, 50, np.int32))
        err[kk] = float(np.sqrt(((r["y"] - x) ** 2).mean()))
    assert err[5] < err[4] < err[3] < 0.25, err


def test_unpack_restores_the_quantised_rows(oracle):
    blob = make_blob()
    x, grp, pos = _rows(96, 11)
    r = oracle.tb_encode(blob, x, grp, pos)
    back = oracle.tb_unpack(blob, grp, pos, r["pay"], r["side"], x)
    assert np.array_equal(back, r["y"])                          # by value: a flat code of -0 decodes to +0
