"""Generates the known-answer file kvx_post_kat.npz from the CPU oracle (oracle/kvx_oracle.c, ysko_kvx_attn_post).

    python tests/golden/make_kvx_post_kat.py

Two seeded cases of the attention block's row epilogue over INT8 rows (RMS norm, partial RoPE, sign-Hadamard-256 rotation,
INT8 rows appended): the shipping shape's head counts at rotary width 64, and a small one at rotary width 128.  Inputs are
bf16 bit patterns; among the rows are an all-zero row and a row of large values.  The file freezes the oracle's behaviour;
the oracle itself is pinned against the reference's kernel on a GPU (tests/test_ref_pin.py).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import kv4_oracle as o          # noqa: E402
from tests.helpers import post_inputs as inputs   # noqa: E402


def run_oracle(d, eps, pos0, rd, max_ctx):
    kvh = d["k_rows"].shape[1]
    k8 = np.zeros((kvh, max_ctx, 256), dtype=np.int8); v8 = np.zeros_like(k8)
    ks = np.zeros((kvh, max_ctx), dtype=np.float32); vs = np.zeros_like(ks)
    q16, gate16 = o.kvx_attn_post(d["q_rows"], d["k_rows"], d["v_rows"], d["qn_w"], d["kn_w"], eps, pos0, d["rope"], rd, max_ctx, k8, ks, v8, vs)
    M = d["q_rows"].shape[0]
    return dict(q16=q16, gate16=gate16, k8=k8[:, pos0:pos0 + M].copy(), v8=v8[:, pos0:pos0 + M].copy(),
                ks=ks[:, pos0:pos0 + M].copy(), vs=vs[:, pos0:pos0 + M].copy())


CASES = {"a": dict(seed=501, M=3, nh=24, kvh=4, rd=64, max_ctx=64, pos0=37, eps=1e-6),
         "b": dict(seed=502, M=2, nh=4, kvh=2, rd=128, max_ctx=32, pos0=5, eps=1e-5)}


def main():
    out = {}
    for name, c in CASES.items():
        d = inputs(c["seed"], c["M"], c["nh"], c["kvh"], c["rd"], c["max_ctx"])
        r = run_oracle(d, c["eps"], c["pos0"], c["rd"], c["max_ctx"])
        for k_, v_ in {**d, **r}.items():
            out[f"{name}_{k_}"] = v_
    np.savez_compressed(os.path.join(HERE, "kvx_post_kat.npz"), **out)
    print("kvx_post_kat.npz", {k_: v_.shape for k_, v_ in out.items() if k_.startswith("a_")})


if __name__ == "__main__":
    main()
