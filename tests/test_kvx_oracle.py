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
