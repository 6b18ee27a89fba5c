"""Generates the known-answer files kv4_kat_*.npz from the CPU oracle (oracle/kv4_oracle.c).

    python tests/golden/make_kv4_kat.py

Each file holds seeded inputs (K/V rows as fp16 bits, Q rows, rope table) and the oracle's outputs: the
packed cache after appending ctx tokens in ragged passes, and the exact attention output of M query rows.
The files freeze the oracle's behaviour; the oracle itself is pinned against the reference's CUDA
kernels on a GPU (tests/test_ref_pin.py).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import kv4_oracle as o          # noqa: E402
from tests.helpers import f16_bits          # noqa: E402
from yasakani_b200 import synth             # noqa: E402

CASES = {
    # name: (shape, ctx already cached, M query rows appended after it, ragged append pass sizes)
    "hd128_ctx97": (synth.Shape(hq=16, hkv=2, hd=128, rd=128, theta=1e6), 97, 3, [1, 30, 2, 33, 31]),
    "hd256_ctx97": (synth.Shape(hq=12, hkv=2, hd=256, rd=64, theta=1e7), 97, 3, [40, 1, 56]),
}


def make(name):
    shape, ctx, M, passes = CASES[name]
    assert sum(passes) == ctx
    max_ctx = 128
    k, v = synth.make_kv(shape, ctx + M, seed=4321)
    q = synth.make_q(shape, M, seed=4321)
    k16, v16, q16 = f16_bits(k), f16_bits(v), f16_bits(q)
    kv = o.KvCache(shape.hkv, shape.hd, max_ctx)
    p = 0
    for n in passes + [M]:
        o.append(kv, p, k16[p:p + n], v16[p:p + n]); p += n
    rope = o.rope_table(max_ctx, shape.theta, shape.rd)
    out = o.attention_exact(q16, kv, ctx, rope, shape.hq, shape.rd, shape.qscale)
    np.savez_compressed(os.path.join(HERE, f"kv4_kat_{name}.npz"), k16=k16, v16=v16, q16=q16, rope=rope, out=out,
                        passes=np.array(passes + [M]), meta=np.array([shape.hq, shape.hkv, shape.hd, shape.rd, ctx, M, max_ctx]),
                        theta=np.float32(shape.theta), **kv.arrays())


if __name__ == "__main__":
    for n in CASES:
        make(n)
        print("wrote", n)
