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
