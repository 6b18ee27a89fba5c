"""Generates the known-answer file kvx_kat.npz from the CPU oracle (oracle/kvx_oracle.c).

    python tests/golden/make_kvx_kat.py

Seeded rows of 256 fp32 values (normal, heavy-tailed, tiny, an all-zero row, a one-hot row, a constant row) and the
oracle's outputs: rotated rows, INT8 payload, scales and the decoded rows.  The file freezes the oracle's behaviour;
the oracle itself is pinned against the reference's probe on a GPU (tests/test_ref_pin.py).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import kv4_oracle as o          # noqa: E402


def rows(seed=77):
    rng = np.random.default_rng(seed)
    x = np.concatenate([
        rng.standard_normal((6, 256)),
        rng.standard_normal((4, 256)) * np.exp(rng.uniform(np.log(0.5), np.log(4.0), (4, 256))),
        rng.standard_cauchy((2, 256)),
        rng.standard_normal((2, 256)) * 1e-30,
        np.zeros((1, 256)),
        np.eye(1, 256, 37) * 3.25,
        np.full((1, 256), -0.75),
        rng.standard_normal((1, 256)) * 3e4,
    ]).astype(np.float32)
    return x


def main():
    x = rows()
    q, sc = o.kvx_encode(x)
    np.savez_compressed(os.path.join(HERE, "kvx_kat.npz"), x=x, sign=o.kvx_sign(), rot=o.kvx_rotate(x), q=q, scales=sc,
                        y=o.kvx_decode(q, sc))
    print("kvx_kat.npz", x.shape)


if __name__ == "__main__":
    main()
