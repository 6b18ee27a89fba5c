"""ctypes binding of the CPU oracle (oracle/kv4_oracle.c) over numpy arrays.

TEST INFRASTRUCTURE, NOT PRODUCT: only tests/, the smoke check and the bench's
CPU-baseline leg import this module.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile the oracle (and, if the reference tree is mounted, oracle/_ref)."""
    so = os.path.join(_HERE, "libkv4_oracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("kv4_oracle.c", "kvx_oracle.c", "tb_oracle.c", "kv4_oracle.h")]
    if force or not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(f) for f in srcs):
        subprocess.run(["make", "-C", _HERE, "libkv4_oracle.so"], check=True, capture_output=True)
    return so


class _Layer(C.Structure):
    _fields_ = [("kq", C.c_void_p), ("kscale", C.c_void_p), ("kzero", C.c_void_p), ("kshadow", C.c_void_p),
                ("vq", C.c_void_p), ("vscale", C.c_void_p), ("vzero", C.c_void_p)]


def lib():
    global _LIB
    if _LIB is None:
        L = C.CDLL(build())
        L.ysko_f32_to_f16.restype = C.c_uint16
        L.ysko_f32_to_f16.argtypes = [C.c_float]
        L.ysko_f16_to_f32.restype = C.c_float
        L.ysko_f16_to_f32.argtypes = [C.c_uint16]
        L.ysko_max_threads.restype = C.c_int
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class KvCache:
    """Packed KV4 cache of one layer in the reference's layout (numpy, host)."""

    def __init__(self, hkv: int, hd: int, max_ctx: int):
        assert max_ctx % 64 == 0 and hd % 32 == 0
        self.hkv, self.hd, self.max_ctx = hkv, hd, max_ctx
        ng = max_ctx // 32
        self.kq = np.zeros((hkv, ng, 32, hd // 2), np.uint8)
        self.kscale = np.zeros((hkv, ng, hd), np.uint16)
        self.kzero = np.zeros((hkv, ng, hd), np.uint16)
        self.kshadow = np.zeros((hkv, max_ctx, hd), np.uint16)
        self.vq = np.zeros((hkv, max_ctx, hd // 2), np.uint8)
        self.vscale = np.zeros((hkv, max_ctx), np.uint16)
        self.vzero = np.zeros((hkv, max_ctx), np.uint16)

    NAMES = ("kq", "kscale", "kzero", "kshadow", "vq", "vscale", "vzero")

    def arrays(self):
        return {n: getattr(self, n) for n in self.NAMES}

    def struct(self):
        return _Layer(*[_p(getattr(self, n)) for n in self.NAMES])


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def bf16_bits_to_f16_bits(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint16)
    out = np.empty_like(b)
    lib().ysko_bf16_to_f16_array(_p(b), _p(out), C.c_size_t(b.size))
    return out


def rope_table(max_ctx: int, theta: float, rd: int) -> np.ndarray:
    out = np.zeros((max_ctx, rd // 2, 2), np.float32)
    lib().ysko_rope_table(_p(out), max_ctx, C.c_float(theta), rd)
    return out


def append(kv: KvCache, pos0: int, k16: np.ndarray, v16: np.ndarray) -> None:
    """k16, v16: uint16 fp16 bits [M][Hkv][HD]."""
    k16 = np.ascontiguousarray(k16, np.uint16)
    v16 = np.ascontiguousarray(v16, np.uint16)
    M = k16.shape[0]
    assert k16.shape == (M, kv.hkv, kv.hd) and v16.shape == k16.shape and pos0 + M <= kv.max_ctx
    s = kv.struct()
    lib().ysko_append(C.byref(s), kv.hkv, kv.hd, kv.max_ctx, pos0, M, _p(k16), _p(v16))


def group_quant(kv: KvCache, pos0: int, M: int) -> None:
    s = kv.struct()
    lib().ysko_group_quant(C.byref(s), kv.hkv, kv.hd, kv.max_ctx, pos0, M)


def attention_partials(q16, kv: KvCache, pos0: int, S: int, rope, hq: int, rd: int, qscale: float, threads: int = 0,
                       shard_start: int = 0, shard_len: int | None = None):
    q16 = np.ascontiguousarray(q16, np.uint16)
    M = q16.shape[0]
    pm = np.zeros((M, S, hq), np.float32)
    pl = np.zeros((M, S, hq), np.float32)
    pacc = np.zeros((M, S, hq, kv.hd), np.float32)
    s = kv.struct()
    lib().ysko_attention_partials_shard(_p(q16), C.byref(s), kv.max_ctx, M, pos0, S, _p(pm), _p(pl), _p(pacc), _p(rope),
                                        kv.hkv, hq, kv.hd, rd, C.c_float(qscale), threads or lib().ysko_max_threads(),
                                        shard_start, kv.max_ctx if shard_len is None else shard_len)
    return pm, pl, pacc


def combine(pm, pl, pacc, g: int, bv=None, gate=None) -> np.ndarray:
    M, S, hq = pm.shape
    hd = pacc.shape[-1]
    o16 = np.zeros((M, hq, hd), np.uint16)
    lib().ysko_combine(_p(np.ascontiguousarray(pm)), _p(np.ascontiguousarray(pl)), _p(np.ascontiguousarray(pacc)),
                       S, M, hq, g, hd, _p(bv), _p(gate), _p(o16))
    return o16


def attention_exact(q16, kv: KvCache, pos0: int, rope, hq: int, rd: int, qscale: float,
                    rows=None, threads: int = 0, wk=None) -> np.ndarray:
    """float32 [M][Hq][HD]; rows=(begin,end) restricts the computed rows (others stay 0).  wk: optional uint8 row -> depth
    table of a tree-shaped pass (row r at position pos0 + wk[r], own key in slot pos0 + r)."""
    q16 = np.ascontiguousarray(q16, np.uint16)
    M = q16.shape[0]
    out = np.zeros((M, hq, kv.hd), np.float32)
    b, e = rows if rows is not None else (0, M)
    s = kv.struct()
    wk = None if wk is None else np.ascontiguousarray(wk, np.uint8)
    lib().ysko_attention_exact_wk(_p(q16), C.byref(s), kv.max_ctx, M, pos0, _p(rope), kv.hkv, hq, kv.hd, rd,
                                  C.c_float(qscale), _p(out), b, e, threads or lib().ysko_max_threads(), _p(wk))
    return out


def xform_a8(o16: np.ndarray, signs: np.ndarray):
    """o16 uint16 fp16 bits [M][n] (n a multiple of 512), signs int8 [n] -> (qx int8 [M][n], alpha float32 [M][n/512])."""
    o16 = np.ascontiguousarray(o16, np.uint16); M = o16.shape[0]; o16 = o16.reshape(M, -1); n = o16.shape[1]
    signs = np.ascontiguousarray(signs, np.int8)
    qx = np.empty((M, n), np.int8); alpha = np.empty((M, n // 512), np.float32)
    lib().ysko_xform_a8(_p(o16), _p(signs), _p(qx), _p(alpha), M, n)
    return qx, alpha


def merge_triples(parts: np.ndarray) -> np.ndarray:
    parts = np.ascontiguousarray(parts, np.float32)
    R, hq, w = parts.shape
    out = np.zeros((hq, w - 2), np.float32)
    lib().ysko_merge_triples(_p(parts), R, hq, w - 2, _p(out))
    return out


def max_threads() -> int:
    return int(lib().ysko_max_threads())


# ---------------------------------------------------------------- Family-B row codec, step 2: trellis rows (tb_oracle.c)
def tb_check_blob(blob: bytes) -> int:
    """0 if the reference's loader would accept the "KVQP v1" blob (src/engine35.cpp:50-53, src/kvq_fast.hpp:52-76)."""
    a = np.frombuffer(blob, np.uint8)
    return int(lib().ysko_tb_check_blob(_p(a), C.c_size_t(a.size)))


def tb_encode(blob: bytes, x: np.ndarray, grp: np.ndarray, pos: np.ndarray):
    """x [rows][256] float32; grp, pos int32 [rows] -> dict(y, fields, pay [rows][40] uint32, side [rows][2] uint32, kb [rows])."""
    a = np.frombuffer(blob, np.uint8)
    x = np.ascontiguousarray(x, np.float32).reshape(-1, 256); rows = x.shape[0]
    grp = np.ascontiguousarray(grp, np.int32); pos = np.ascontiguousarray(pos, np.int32)
    y = np.empty_like(x); fields = np.empty((rows, 256), np.uint8); pay = np.empty((rows, 40), np.uint32)
    side = np.empty((rows, 2), np.uint32); kb = np.empty(rows, np.int32)
    lib().ysko_tb_encode(_p(a), _p(x), _p(grp), _p(pos), rows, _p(y), _p(fields), _p(pay), _p(side), _p(kb))
    return {"y": y, "fields": fields, "pay": pay, "side": side, "kb": kb}


def tb_unpack(blob: bytes, grp, pos, pay: np.ndarray, side: np.ndarray, yin: np.ndarray) -> np.ndarray:
    """Packed rows back to values (tba_unpack_kernel, src/kvq_attn.cuh:39-72); pay uint32 [rows][stride_words]."""
    a = np.frombuffer(blob, np.uint8)
    grp = np.ascontiguousarray(grp, np.int32); pos = np.ascontiguousarray(pos, np.int32)
    pay = np.ascontiguousarray(pay, np.uint32); side = np.ascontiguousarray(side, np.uint32)
    yin = np.ascontiguousarray(yin, np.float32).reshape(-1, 256); y = np.empty_like(yin)
    lib().ysko_tb_unpack(_p(a), _p(grp), _p(pos), _p(pay), pay.shape[1], _p(side), _p(yin), _p(y), yin.shape[0])
    return y


def tb_decode_fields(blob: bytes, g: int, pay: np.ndarray, scale: float) -> np.ndarray:
    a = np.frombuffer(blob, np.uint8)
    pay = np.ascontiguousarray(pay, np.uint32); xq = np.empty(256, np.float32)
    lib().ysko_tb_decode_fields(_p(a), int(g), _p(pay), C.c_float(scale), _p(xq))
    return xq


# ---------------------------------------------------------------- Family-B row codec, step 1 (kvx_oracle.c)
def kvx_sign() -> np.ndarray:
    L = lib(); L.ysko_kvx_sign.restype = C.c_float; L.ysko_kvx_sign.argtypes = [C.c_int]
    return np.array([L.ysko_kvx_sign(d) for d in range(256)], dtype=np.float32)


def kvx_rotate(x: np.ndarray, inverse: bool = False) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 256)
    y = np.empty_like(x)
    lib().ysko_kvx_rotate(_p(x), _p(y), C.c_long(x.shape[0]), C.c_int(1 if inverse else 0))
    return y


def kvx_encode(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 256)
    q = np.empty(x.shape, dtype=np.int8); sc = np.empty(x.shape[0], dtype=np.float32)
    lib().ysko_kvx_encode(_p(x), _p(q), _p(sc), C.c_long(x.shape[0]))
    return q, sc


def kvx_attn_post(q_rows, k_rows, v_rows, qn_w, kn_w, eps: float, pos0: int, rope, rd: int, max_ctx: int, k8, ks, v8, vs):
    """ysko_kvx_attn_post: rows as bf16 bit patterns (uint16) -- q_rows [M][nh][512], k_rows / v_rows [M][kvh][256]; the
    INT8 row caches k8 / v8 [kvh][max_ctx][256] and ks / vs [kvh][max_ctx] are updated in place at pos0 .. pos0 + M - 1.
    Returns (q16, gate16) as bf16 bit patterns [M][nh][256]."""
    q_rows = np.ascontiguousarray(q_rows, dtype=np.uint16); k_rows = np.ascontiguousarray(k_rows, dtype=np.uint16)
    v_rows = np.ascontiguousarray(v_rows, dtype=np.uint16)
    qn_w = np.ascontiguousarray(qn_w, dtype=np.uint16); kn_w = np.ascontiguousarray(kn_w, dtype=np.uint16)
    rope = np.ascontiguousarray(rope, dtype=np.float32)
    M, nh = q_rows.shape[0], q_rows.shape[1]; kvh = k_rows.shape[1]
    assert q_rows.shape == (M, nh, 512) and k_rows.shape == (M, kvh, 256) and v_rows.shape == (M, kvh, 256)
    assert k8.dtype == np.int8 and v8.dtype == np.int8 and ks.dtype == np.float32 and vs.dtype == np.float32
    assert k8.shape == (kvh, max_ctx, 256) and k8.flags.c_contiguous and v8.flags.c_contiguous and pos0 + M <= max_ctx
    q16 = np.empty((M, nh, 256), dtype=np.uint16); gate16 = np.empty((M, nh, 256), dtype=np.uint16)
    lib().ysko_kvx_attn_post(_p(q_rows), _p(k_rows), _p(v_rows), _p(qn_w), _p(kn_w), C.c_float(eps), int(M), int(pos0), _p(rope), int(rd),
                             int(nh), int(kvh), int(max_ctx), _p(q16), _p(gate16), _p(k8), _p(ks), _p(v8), _p(vs))
    return q16, gate16


def kvx_decode(q: np.ndarray, sc: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.int8).reshape(-1, 256); sc = np.ascontiguousarray(sc, dtype=np.float32)
    y = np.empty(q.shape, dtype=np.float32)
    lib().ysko_kvx_decode(_p(q), _p(sc), _p(y), C.c_long(q.shape[0]))
    return y


def kv8_attention_exact(q: np.ndarray, k8: np.ndarray, v8: np.ndarray, ks: np.ndarray, vs: np.ndarray, pos0: int, qscale: float = 0.0625) -> np.ndarray:
    """q [M, nh, 256] fp32 (rotated), k8/v8 [kvh, max_ctx, 256] int8, ks/vs [kvh, max_ctx] -> [M, nh, 256] in the rotated basis."""
    q = np.ascontiguousarray(q, dtype=np.float32); k8 = np.ascontiguousarray(k8, dtype=np.int8); v8 = np.ascontiguousarray(v8, dtype=np.int8)
    ks = np.ascontiguousarray(ks, dtype=np.float32); vs = np.ascontiguousarray(vs, dtype=np.float32)
    M, nh, _ = q.shape; kvh, max_ctx, _ = k8.shape
    out = np.empty_like(q)
    lib().ysko_kv8_attention_exact(_p(q), _p(k8), _p(v8), _p(ks), _p(vs), C.c_int(max_ctx), C.c_int(M), C.c_int(pos0), C.c_int(kvh),
                                   C.c_int(nh), C.c_float(qscale), _p(out))
    return out


def rows_attention_exact(q: np.ndarray, k: np.ndarray, v: np.ndarray, pos0: int, qscale: float = 0.0625) -> np.ndarray:
    """q [M, nh, 256] fp32, k / v [kvh, max_ctx, 256] fp32 rows -> [M, nh, 256] (ysko_rows_attention_exact)."""
    q = np.ascontiguousarray(q, dtype=np.float32); k = np.ascontiguousarray(k, dtype=np.float32); v = np.ascontiguousarray(v, dtype=np.float32)
    M, nh = q.shape[0], q.shape[1]; kvh, max_ctx = k.shape[0], k.shape[1]
    assert q.shape == (M, nh, 256) and k.shape == (kvh, max_ctx, 256) and v.shape == k.shape and pos0 + M <= max_ctx
    out = np.empty((M, nh, 256), dtype=np.float32)
    lib().ysko_rows_attention_exact(_p(q), _p(k), _p(v), int(max_ctx), int(M), int(pos0), int(kvh), int(nh), C.c_float(qscale), _p(out))
    return out
