"""Host-side mirror of the reference's Family-B row codec, step 1 (src/kvx_codec.cuh): sign-Hadamard-256 rotation and
INT8 rows with one fp32 scale per row.  Same rules as kv4.py: torch tensors are device memory only, every call is
enqueue-only on torch's current stream, all arithmetic happens in libyskn_kv4.so, no fallback."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check, Kv8AttnArgsC
from .kv4 import _ptr, _stream, _dtype_code


def _rows(t: torch.Tensor) -> int:
    if t.numel() % 256:
        raise ValueError("rows are 256 values long")
    return t.numel() // 256


def rotate(x: torch.Tensor, inverse: bool = False, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """kvx_rotate (src/kvx_codec.cuh:35-49) on fp32 rows."""
    if x.dtype != torch.float32:
        raise TypeError("yskn_kvx_rotate takes fp32 rows")
    out = torch.empty_like(x) if out is None else out
    check(_lib.load().yskn_kvx_rotate(_ptr(x), _ptr(out), _rows(x), 1 if inverse else 0, _stream(stream)), "yskn_kvx_rotate")
    return out


def encode(x: torch.Tensor, q8: torch.Tensor | None = None, scales: torch.Tensor | None = None, stream=None):
    """Rotation + kvx_store (src/kvx_codec.cuh:50-70): returns (q8 int8 [rows, 256], scales fp32 [rows])."""
    rows = _rows(x)
    q8 = torch.empty((rows, 256), dtype=torch.int8, device=x.device) if q8 is None else q8
    scales = torch.empty((rows,), dtype=torch.float32, device=x.device) if scales is None else scales
    check(_lib.load().yskn_kvx_encode(_ptr(x), _dtype_code(x), _ptr(q8), _ptr(scales), rows, _stream(stream)), "yskn_kvx_encode")
    return q8, scales


def decode(q8: torch.Tensor, scales: torch.Tensor, dtype=torch.float32, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """(float)q * scale, then the inverse rotation (src/kvx_probe.cu:15-19)."""
    rows = _rows(q8)
    out = torch.empty((rows, 256), dtype=dtype, device=q8.device) if out is None else out
    check(_lib.load().yskn_kvx_decode(_ptr(q8), _ptr(scales), _ptr(out), _dtype_code(out), rows, _stream(stream)), "yskn_kvx_decode")
    return out


def launch_attn_post(q_rows, k_rows, v_rows, qn_w, kn_w, eps: float, d_pos, rope, rd: int, q16, gate16, k8, ks, v8, vs,
                     pm: bool = True, stream=None) -> None:
    """launch_q35_attn_post (src/q35_kernels.cu:1013-1069) from the bf16 projection rows on: RMS norm, partial RoPE and
    rotation of the query and key heads, INT8 rows of keys and values appended at *d_pos + token, gate copied.
    q_rows bf16 [M, nh, 512]; k_rows / v_rows bf16 [M, kvh, 256]; k8 / v8 int8 [kvh, max_ctx, 256]; ks / vs fp32 [kvh, max_ctx]."""
    M, nh = q_rows.shape[0], q_rows.shape[1]
    kvh, max_ctx = k8.shape[0], k8.shape[1]
    for t in (q_rows, k_rows, v_rows, qn_w, kn_w, q16, gate16):
        if t.dtype != torch.bfloat16:
            raise TypeError("yskn_kvx_attn_post takes bf16 rows and norm weights")
    if tuple(q_rows.shape) != (M, nh, 512) or tuple(k_rows.shape) != (M, kvh, 256) or tuple(v_rows.shape) != (M, kvh, 256):
        raise ValueError("q_rows [M, nh, 512], k_rows / v_rows [M, kvh, 256]")
    a = _lib.KvxAttnPostArgsC(_ptr(q_rows), _ptr(k_rows), _ptr(v_rows), _ptr(qn_w), _ptr(kn_w), eps, M, _ptr(d_pos),
                              _ptr(rope) if rope is not None else None, rd, _ptr(q16), _ptr(gate16), _ptr(k8), _ptr(v8), _ptr(ks), _ptr(vs),
                              max_ctx, nh, kvh, 1 if pm else 0)
    check(_lib.load().yskn_kvx_attn_post(C.byref(a), _stream(stream)), "yskn_kvx_attn_post")


def probe(x: np.ndarray):
    """The reference's yskn_kvx_probe contract over host arrays: (q, scales, y)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 256)
    rows = x.shape[0]
    q = np.empty((rows, 256), dtype=np.int8); sc = np.empty(rows, dtype=np.float32); y = np.empty_like(x)
    rc = _lib.load().yskn_kvx_probe(x.ctypes.data_as(C.c_void_p), q.ctypes.data_as(C.c_void_p), sc.ctypes.data_as(C.c_void_p),
                                    y.ctypes.data_as(C.c_void_p), rows)
    if rc == -1 and (rows <= 0 or rows % 2):
        raise ValueError("yskn_kvx_probe takes an even, positive number of rows")
    check(rc, "yskn_kvx_probe")
    return q, sc, y


def _dp(t):
    return None if t is None else t.data_ptr()


def launch_kv8_attention(q16: torch.Tensor, k8: torch.Tensor, v8: torch.Tensor, ks: torch.Tensor, vs: torch.Tensor, M: int,
                         d_pos: torch.Tensor, splits: int, pm: torch.Tensor, pl: torch.Tensor, pacc: torch.Tensor, nh: int,
                         qscale: float = 0.0625, stream=None) -> None:
    """launch_q35_attention, INT8 branch (src/q35_kernels.cu:1176-1281): k8/v8 [kvh, max_ctx, 256] int8, ks/vs [kvh, max_ctx]."""
    kvh, max_ctx = k8.shape[0], k8.shape[1]
    for t in (q16, k8, v8, ks, vs, d_pos, pm, pl, pacc):
        assert t.is_cuda and t.is_contiguous()
    a = Kv8AttnArgsC(_dp(q16), _dp(k8), _dp(v8), _dp(ks), _dp(vs), max_ctx, M, _dp(d_pos), splits, _dp(pm), _dp(pl), _dp(pacc), kvh, nh, qscale)
    check(_lib.load().yskn_kv8_attention(C.byref(a), _dtype_code(q16), _stream(stream)), "yskn_kv8_attention")


def launch_kv8_attention_tc(q16: torch.Tensor, k8: torch.Tensor, v8: torch.Tensor, ks: torch.Tensor, vs: torch.Tensor, M: int,
                            d_pos: torch.Tensor, splits: int, pm: torch.Tensor, pl: torch.Tensor, pacc: torch.Tensor, nh: int,
                            qscale: float = 0.0625, stream=None) -> None:
    """Many rows over INT8 rows on the tcgen05 kernel (launch_q35_atx, src/q35_atx.cu:92-793): same arguments and partials."""
    kvh, max_ctx = k8.shape[0], k8.shape[1]
    for t in (q16, k8, v8, ks, vs, d_pos, pm, pl, pacc):
        assert t.is_cuda and t.is_contiguous()
    a = Kv8AttnArgsC(_dp(q16), _dp(k8), _dp(v8), _dp(ks), _dp(vs), max_ctx, M, _dp(d_pos), splits, _dp(pm), _dp(pl), _dp(pacc), kvh, nh, qscale)
    check(_lib.load().yskn_kv8_attention_tc(C.byref(a), _dtype_code(q16), _stream(stream)), "yskn_kv8_attention_tc")


def launch_kv8_combine(pm, pl, pacc, splits: int, M: int, nh: int, o16: torch.Tensor, gate: torch.Tensor | None = None,
                       inverse_rotate: bool = True, stream=None) -> None:
    """Split merge, inverse rotation, rounding, optional sigmoid gate (src/q35_kernels.cu:1400-1424)."""
    check(_lib.load().yskn_kv8_combine(_ptr(pm), _ptr(pl), _ptr(pacc), splits, M, nh, _ptr(gate), _ptr(o16), _dtype_code(o16),
                                       1 if inverse_rotate else 0, _stream(stream)), "yskn_kv8_combine")


# ---------------------------------------------------------------- step 2: trellis rows (src/kvq_gpu.cuh, src/kvq_fast.cuh)
class TrellisProfile:
    """A "KVQP v1" profile blob checked with the reference loader's rules and uploaded to the current device."""

    def __init__(self, blob: bytes):
        host = np.frombuffer(blob, np.uint8)
        nm = C.c_int(0)
        check(_lib.load().yskn_tb_blob_info(host.ctypes.data, host.size, C.byref(nm)), "yskn_tb_blob_info")
        self.nm = nm.value
        self.dev = torch.from_numpy(host.copy()).cuda()


def tb_encode(profile: TrellisProfile, x: torch.Tensor, grp: torch.Tensor, pos: torch.Tensor, pay_stride: int = 160, stream=None):
    """launch_tb_fast (src/kvq_fast.cuh:242-255) over fp32 rows x [rows][256]: returns (y, pay uint8 [rows][pay_stride],
    side int32-bits [rows][2]); grp, pos int32 device tensors [rows]."""
    rows = _rows(x)
    assert x.dtype == torch.float32 and grp.dtype == torch.int32 and pos.dtype == torch.int32
    L = _lib.load()
    y = torch.empty_like(x)
    pay = torch.zeros((rows, pay_stride), dtype=torch.uint8, device=x.device)
    side = torch.zeros((rows, 2), dtype=torch.int32, device=x.device)
    scratch = torch.empty(int(L.yskn_tb_scratch_bytes(rows, profile.nm)), dtype=torch.uint8, device=x.device)
    check(L.yskn_tb_encode(_ptr(profile.dev), profile.nm, _ptr(x), _ptr(grp), _ptr(pos), rows, _ptr(y), _ptr(pay), pay_stride, _ptr(side),
                           _ptr(scratch), scratch.numel(), _stream(stream)), "yskn_tb_encode")
    return y, pay, side


def tb_decode(profile: TrellisProfile, pay: torch.Tensor, side: torch.Tensor, grp: torch.Tensor, pos: torch.Tensor, yin: torch.Tensor | None = None,
              stream=None) -> torch.Tensor:
    """tba_unpack_kernel (src/kvq_attn.cuh:39-72): payload rows [rows][stride] + side words -> fp32 rows [rows][256]."""
    rows = pay.shape[0]
    y = torch.empty((rows, 256), dtype=torch.float32, device=pay.device)
    check(_lib.load().yskn_tb_decode(_ptr(profile.dev), _ptr(grp), _ptr(pos), _ptr(pay), pay.shape[1], _ptr(side),
                                    _ptr(yin) if yin is not None else None, _ptr(y), rows, _stream(stream)), "yskn_tb_decode")
    return y


def launch_tb_attention(profile: TrellisProfile, q16, k_pay, k_side, v_pay, v_side, grp_k, grp_v, M: int, d_pos, splits: int, pm, pl, pacc, nh: int,
                        k_plain=None, v_plain=None, qscale: float = 0.0625, stream=None) -> None:
    """Decode attention straight over packed trellis rows (the reference's launch_q35_atxpk for a few rows): k_pay / v_pay uint8
    [kvh, max_ctx, stride], k_side / v_side int32-bits [kvh, max_ctx, 2], grp_k / grp_v int32 [kvh]; rows the profile leaves
    unpacked come from k_plain / v_plain fp32 [kvh, max_ctx, 256].  Partials as launch_kv8_attention."""
    kvh, max_ctx, stride = k_pay.shape
    a = _lib.TbAttnArgsC(_ptr(q16), _ptr(profile.dev), _ptr(k_pay), _ptr(v_pay), stride, _ptr(k_side), _ptr(v_side), _ptr(grp_k), _ptr(grp_v),
                         _ptr(k_plain) if k_plain is not None else None, _ptr(v_plain) if v_plain is not None else None,
                         max_ctx, M, _ptr(d_pos), splits, _ptr(pm), _ptr(pl), _ptr(pacc), kvh, nh, qscale)
    check(_lib.load().yskn_tb_attention(C.byref(a), _dtype_code(q16), _stream(stream)), "yskn_tb_attention")
