"""Generator of a SYNTHETIC "KVQP v1" profile blob for the trellis ("CDQ") KV codec.

The shipping blob (kvq_u5.bin) lives in the model folder, not in the reference repository, so results over this blob can
only be self-consistent with the reference's code, never with shipped tables.  The layout is the one the reference's
loader and kernels read (src/engine35.cpp:50-53, src/kvq_gpu.cuh:57-68,89-93, src/kvq_fast.hpp:52-76):

  header (96 bytes): "KVQP", u16 version 1, u16 header size 96, u32 total size, u16 D 256 @16, u16 layers 16 @18,
                     u16 kv heads 4 @20, u16 tables @22, u16 multipliers @24, u32 groups 128 @28, u32 offsets of the
                     multipliers @32, of the table offsets @36, of the group offsets @40
  multipliers:       f32[nm]                       scale = fp16(rms * multiplier)
  table record:      u8 L 8, u8 -, u8 chain 64, u8 F 8, f32 gain, 4 bytes, i16 code[256] (|code| <= 1100)
  group record:      u8 mode (0 trellis, 1 flat), u8 bits per step (3/4/5), u8 table, u8 guard (positions below stay
                     unpacked), u8 low-rank count (0..2), u8 has-mean, 2 bytes, then f16 mean[256] and f16 U[m][256]
  group index g = (layer * 4 + kv_head) * 2 + kind (0 = K, 1 = V).

Codes are the sorted quantiles of a Gaussian scaled to the reference's integer grid (x / s * 256), shuffled by a fixed
permutation of the 256 states so that the shift-register structure has to be honoured.  `python make_kvqp_blob.py`
writes tests/golden/kvqp_synthetic.bin; tests import make_blob().
"""
from __future__ import annotations

import os
import struct

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def make_blob(seed: int = 2026, nm: int = 5) -> bytes:
    rng = np.random.default_rng(seed)
    ngrp, nt = 128, 3
    mult = np.linspace(0.7, 1.5, nm).astype(np.float32)
    # three code tables, for 3, 4 and 5 bits per step
    tables = []
    for t, kk in enumerate((3, 4, 5)):
        q = np.sort(rng.standard_normal(256)).astype(np.float64)
        q = q / np.abs(q).max() * 3.2                              # +-3.2 rms
        code = np.clip(np.rint(q * 256.0), -1100, 1100).astype(np.int16)
        code = code[rng.permutation(256)]
        gain = np.float32(1.0 + 0.01 * t)
        tables.append(struct.pack("<BBBBf4x", 8, 0, 64, 8, float(gain)) + code.astype("<i2").tobytes())
    groups = []
    for g in range(ngrp):
        kind = g & 1
        mode = 1 if g % 16 == 15 else 0                            # a few flat groups
        kk = (4, 5, 4, 5, 3, 4, 5, 4)[(g // 2) % 8]
        tix = {3: 0, 4: 1, 5: 2}[kk]
        guard = 4 if g % 8 == 0 else 0
        m = (0, 1, 2)[g % 3]
        has_mu = 1 if g % 4 != 3 else 0
        rec = struct.pack("<BBBBBB2x", mode, kk, tix, guard, m, has_mu)
        if has_mu:
            rec += (rng.standard_normal(256) * 0.2).astype(np.float16).tobytes()
        for _ in range(m):
            u = rng.standard_normal(256); u /= np.linalg.norm(u)
            rec += u.astype(np.float16).tobytes()
        groups.append(rec)
    off = 96
    off_m = off; off += 4 * nm
    off_t = off; off += 4 * nt
    off_g = off; off += 4 * ngrp
    tab_off = []
    for t in tables:
        tab_off.append(off); off += len(t)
    grp_off = []
    for r in groups:
        grp_off.append(off); off += len(r)
    total = off
    hdr = bytearray(96)
    hdr[0:4] = b"KVQP"
    struct.pack_into("<HHI", hdr, 4, 1, 96, total)
    struct.pack_into("<HHHHH", hdr, 16, 256, 16, 4, nt, nm)
    struct.pack_into("<IIII", hdr, 28, ngrp, off_m, off_t, off_g)
    blob = bytes(hdr) + mult.astype("<f4").tobytes() + struct.pack(f"<{nt}I", *tab_off) + struct.pack(f"<{ngrp}I", *grp_off)
    blob += b"".join(tables) + b"".join(groups)
    assert len(blob) == total
    return blob


if __name__ == "__main__":
    b = make_blob()
    with open(os.path.join(HERE, "kvqp_synthetic.bin"), "wb") as f:
        f.write(b)
    print(len(b), "bytes")
