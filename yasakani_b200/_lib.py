"""ctypes view of libyskn_kv4.so: the structs and prototypes of include/yskn_kv4_abi.h.

There is no fallback: if the library is missing or an entry fails, callers get an exception.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

F16, BF16, F32 = 0, 1, 2
ALGO_AUTO, ALGO_SCALAR, ALGO_MMA = 0, 1, 2


class KvLayerC(C.Structure):          # yskn_kv_layer
    _fields_ = [("kq", C.c_void_p), ("kscale", C.c_void_p), ("kzero", C.c_void_p), ("kshadow", C.c_void_p),
                ("vq", C.c_void_p), ("vscale", C.c_void_p), ("vzero", C.c_void_p)]


class KvQuantArgsC(C.Structure):      # yskn_kv_quant_args
    _fields_ = [("kv", KvLayerC), ("d_pos", C.c_void_p), ("M", C.c_int), ("max_ctx", C.c_int)]


class AttnGArgsC(C.Structure):        # yskn_attn_g_args
    _fields_ = [("q16", C.c_void_p), ("kv", KvLayerC), ("max_ctx", C.c_int), ("M", C.c_int), ("d_pos", C.c_void_p),
                ("splits", C.c_int), ("pm", C.c_void_p), ("pl", C.c_void_p), ("pacc", C.c_void_p), ("rope", C.c_void_p),
                ("kvh", C.c_int), ("nh", C.c_int), ("qscale", C.c_float)]


class AttnGCombineArgsC(C.Structure):  # yskn_attn_g_combine_args
    _fields_ = [("pm", C.c_void_p), ("pl", C.c_void_p), ("pacc", C.c_void_p), ("splits", C.c_int), ("M", C.c_int),
                ("bv", C.c_void_p), ("o16", C.c_void_p), ("gate", C.c_void_p), ("nh", C.c_int), ("g", C.c_int)]


class KvAppendArgsC(C.Structure):     # yskn_kv_append_args
    _fields_ = [("k_in", C.c_void_p), ("v_in", C.c_void_p), ("in_dtype", C.c_int), ("kv", KvLayerC),
                ("d_pos", C.c_void_p), ("M", C.c_int), ("max_ctx", C.c_int), ("kvh", C.c_int), ("hd", C.c_int)]


class Kv8AttnArgsC(C.Structure):
    _fields_ = [("q16", C.c_void_p), ("k8", C.c_void_p), ("v8", C.c_void_p), ("ks", C.c_void_p), ("vs", C.c_void_p),
                ("max_ctx", C.c_int), ("M", C.c_int), ("d_pos", C.c_void_p), ("splits", C.c_int),
                ("pm", C.c_void_p), ("pl", C.c_void_p), ("pacc", C.c_void_p), ("kvh", C.c_int), ("nh", C.c_int), ("qscale", C.c_float)]


class KvxAttnPostArgsC(C.Structure):  # yskn_kvx_attn_post_args
    _fields_ = [("q_rows", C.c_void_p), ("k_rows", C.c_void_p), ("v_rows", C.c_void_p), ("qn_w", C.c_void_p), ("kn_w", C.c_void_p),
                ("eps", C.c_float), ("M", C.c_int), ("d_pos", C.c_void_p), ("rope", C.c_void_p), ("rd", C.c_int),
                ("q16", C.c_void_p), ("gate16", C.c_void_p), ("k8", C.c_void_p), ("v8", C.c_void_p), ("ks", C.c_void_p), ("vs", C.c_void_p),
                ("max_ctx", C.c_int), ("nh", C.c_int), ("kvh", C.c_int), ("pm", C.c_int)]


class TbAttnArgsC(C.Structure):       # yskn_tb_attn_args
    _fields_ = [("q16", C.c_void_p), ("blob", C.c_void_p), ("k_pay", C.c_void_p), ("v_pay", C.c_void_p), ("pay_stride", C.c_int),
                ("k_side", C.c_void_p), ("v_side", C.c_void_p), ("grp_k", C.c_void_p), ("grp_v", C.c_void_p),
                ("k_plain", C.c_void_p), ("v_plain", C.c_void_p), ("max_ctx", C.c_int), ("M", C.c_int), ("d_pos", C.c_void_p), ("splits", C.c_int),
                ("pm", C.c_void_p), ("pl", C.c_void_p), ("pacc", C.c_void_p), ("kvh", C.c_int), ("nh", C.c_int), ("qscale", C.c_float)]


class AttnExtC(C.Structure):          # yskn_kv4_attn_ext
    _fields_ = [("early", C.c_int), ("splits_short", C.c_int), ("long_len", C.c_int), ("wk", C.c_void_p)]


class MsRowsC(C.Structure):           # yskn_kv4_ms_rows
    _fields_ = [("pos", C.c_void_p), ("slot", C.c_void_p), ("layers", C.c_void_p), ("maps", C.c_void_p), ("n_slots", C.c_int)]


class PeerExchangeC(C.Structure):     # yskn_kv4_peer_exchange
    _fields_ = [("buf", C.c_void_p * 8), ("world", C.c_int), ("rank", C.c_int)]


# name -> (restype, argtypes); every symbol include/yskn_kv4_abi.h declares
PROTOTYPES = {
    "yskn_kv4_last_error": (C.c_char_p, []),
    "yskn_kv4_build_info": (C.c_char_p, []),
    "yskn_kv4_set_algo": (C.c_int, [C.c_int]),
    "yskn_kv4_device_status": (C.c_int, [C.POINTER(C.c_int)]),
    "yskn_kv4_rope_table": (C.c_int, [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_void_p]),
    "yskn_kv4_copy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "yskn_kv4_append": (C.c_int, [C.POINTER(KvAppendArgsC), C.c_void_p]),
    "yskn_kv4_group_quant": (C.c_int, [C.POINTER(KvQuantArgsC), C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_attention": (C.c_int, [C.POINTER(AttnGArgsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_attention_ex": (C.c_int, [C.POINTER(AttnGArgsC), C.POINTER(AttnExtC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_decode_ex": (C.c_int, [C.POINTER(AttnGArgsC), C.POINTER(AttnGCombineArgsC), C.POINTER(AttnExtC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_attention_shard_ex": (C.c_int, [C.POINTER(AttnGArgsC), C.POINTER(AttnExtC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_ms_maps_bytes": (C.c_size_t, [C.c_int]),
    "yskn_kv4_ms_prepare": (C.c_int, [C.POINTER(KvLayerC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "yskn_kv4_attention_ms": (C.c_int, [C.POINTER(AttnGArgsC), C.POINTER(MsRowsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_attention_shard": (C.c_int, [C.POINTER(AttnGArgsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_decode": (C.c_int, [C.POINTER(AttnGArgsC), C.POINTER(AttnGCombineArgsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_decode_shard_triple": (C.c_int, [C.POINTER(AttnGArgsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "yskn_kv4_combine": (C.c_int, [C.POINTER(AttnGCombineArgsC), C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_xform_a8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_prefill": (C.c_int, [C.POINTER(AttnGArgsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "yskn_kv4_set_tc_workspace": (C.c_int, [C.c_void_p, C.c_size_t]),
    "yskn_kv4_tc_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "yskn_kv4_attention_tc": (C.c_int, [C.POINTER(AttnGArgsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "yskn_kv4_prefill_tc": (C.c_int, [C.POINTER(AttnGArgsC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_size_t, C.c_int, C.c_void_p]),
    "yskn_kv4_set_peer_wait_polls": (C.c_int, [C.c_uint]),
    "yskn_kv4_exchange_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "yskn_kv4_push_triple": (C.c_int, [C.POINTER(AttnGCombineArgsC), C.c_int, C.POINTER(PeerExchangeC), C.c_void_p]),
    "yskn_kv4_exchange_merge": (C.c_int, [C.POINTER(AttnGCombineArgsC), C.c_int, C.c_int, C.POINTER(PeerExchangeC), C.c_void_p]),
    "yskn_kv4_merge_pushed": (C.c_int, [C.POINTER(PeerExchangeC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_int, C.c_void_p]),
    "yskn_kv4_local_triple": (C.c_int, [C.POINTER(AttnGCombineArgsC), C.c_int, C.c_void_p, C.c_void_p]),
    "yskn_kv4_merge_triples": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_int, C.c_void_p]),
    "yskn_kv4_decode_noalloc": (C.c_int, [C.c_void_p, C.POINTER(KvLayerC), C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_void_p]),
    "yskn_kvx_rotate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p]),
    "yskn_kvx_encode": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]),
    "yskn_kvx_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_longlong, C.c_void_p]),
    "yskn_kvx_probe": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "yskn_kvx_attn_post": (C.c_int, [C.POINTER(KvxAttnPostArgsC), C.c_void_p]),
    "yskn_tb_attention": (C.c_int, [C.POINTER(TbAttnArgsC), C.c_int, C.c_void_p]),
    "yskn_tb_blob_info": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_int)]),
    "yskn_tb_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "yskn_tb_scratch_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "yskn_tb_encode": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                 C.c_void_p, C.c_size_t, C.c_void_p]),
    "yskn_kv8_attention": (C.c_int, [C.POINTER(Kv8AttnArgsC), C.c_int, C.c_void_p]),
    "yskn_kv8_attention_tc": (C.c_int, [C.POINTER(Kv8AttnArgsC), C.c_int, C.c_void_p]),
    "yskn_kv8_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "yskn_kv4_attention_host": (C.c_int, [C.c_void_p, C.POINTER(KvLayerC), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                          C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_int,
                                          C.c_void_p]),
}

_LIB = None


class Kv4Error(RuntimeError):
    pass


def lib_path() -> str:
    return _build.LIB


def load():
    """Load the CUDA library (building it first if sources are newer). Raises if that is impossible."""
    global _LIB
    if _LIB is None:
        path = _build.LIB
        if not os.path.exists(path) or os.environ.get("YSKN_KV4_REBUILD"):
            path = _build.build()
        L = C.CDLL(path)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(L, name)          # AttributeError here = header and library disagree
            fn.restype, fn.argtypes = res, args
        _LIB = L
    return _LIB


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().yskn_kv4_last_error().decode(errors="replace")
        raise Kv4Error(f"{what} failed (code {rc}): {msg}")
