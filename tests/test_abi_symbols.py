"""The C-ABI library loads on a CPU-only machine and exports every symbol the header declares."""
import ctypes
import os
import re

from yasakani_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "yskn_kv4_abi.h")).read()
    return sorted(set(re.findall(r"YSKN_KV4_API\s+[\w\s\*]+?\b(yskn_(?:kv[48x]|tb)_\w+)\s*\(", text)))


def test_header_and_binding_table_agree():
    syms = declared_symbols()
    assert len(syms) >= 12
    assert sorted(_lib.PROTOTYPES) == syms


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    L = ctypes.CDLL(path)
    for s in declared_symbols():
        assert hasattr(L, s), s
    L.yskn_kv4_build_info.restype = ctypes.c_char_p
    assert b"sm_100a" in L.yskn_kv4_build_info()


def test_struct_layouts_match_the_reference_structs():
    # KvLayer: 7 pointers (src/post_kernels.hpp:7-15); AttnGArgs (src/args.hpp:14-15); AttnGCombineArgs (:16-17)
    assert ctypes.sizeof(_lib.KvLayerC) == 56
    assert _lib.AttnGArgsC.max_ctx.offset == 64 and _lib.AttnGArgsC.d_pos.offset == 72 and _lib.AttnGArgsC.rope.offset == 112
    assert _lib.AttnGArgsC.qscale.offset == 128 and ctypes.sizeof(_lib.AttnGArgsC) == 136
    assert _lib.AttnGCombineArgsC.splits.offset == 24 and _lib.AttnGCombineArgsC.bv.offset == 32
    assert _lib.AttnGCombineArgsC.g.offset == 60 and ctypes.sizeof(_lib.AttnGCombineArgsC) == 64
    assert _lib.KvQuantArgsC.d_pos.offset == 56 and ctypes.sizeof(_lib.KvQuantArgsC) == 72
    # this library's own structs: the ctypes mirrors against the C compiler's layout of include/yskn_kv4_abi.h
    assert _lib.KvxAttnPostArgsC.d_pos.offset == 48 and _lib.KvxAttnPostArgsC.q16.offset == 72 and _lib.KvxAttnPostArgsC.pm.offset == 132
    assert ctypes.sizeof(_lib.KvxAttnPostArgsC) == 136
    assert _lib.TbAttnArgsC.k_side.offset == 40 and _lib.TbAttnArgsC.d_pos.offset == 96 and _lib.TbAttnArgsC.qscale.offset == 144
    assert ctypes.sizeof(_lib.TbAttnArgsC) == 152


def test_argument_rejection_needs_no_gpu():
    L = _lib.load()
    assert L.yskn_kv4_set_algo(99) == -1 and b"unknown algorithm" in L.yskn_kv4_last_error()
    assert L.yskn_kv4_attention(None, 6, 256, 64, 0, None) == -1 and b"null argument" in L.yskn_kv4_last_error()
    assert L.yskn_kv4_rope_table(None, 64, 1e6, 64, None) == -1
    assert L.yskn_kv4_copy(None, None, 0, None) == 0 and L.yskn_kv4_copy(None, None, 16, None) == -1
    assert L.yskn_kv4_copy(ctypes.c_void_p(16), ctypes.c_void_p(32), 24, None) == -1 and b"multiples of 16" in L.yskn_kv4_last_error()
    assert L.yskn_kvx_attn_post(None, None) == -1 and b"null argument" in L.yskn_kv4_last_error()
    assert L.yskn_tb_attention(None, 0, None) == -1 and b"null argument" in L.yskn_kv4_last_error()
    bad = _lib.KvxAttnPostArgsC()
    assert L.yskn_kvx_attn_post(ctypes.byref(bad), None) == 0          # M = 0: nothing to do
    bad.M = 1
    assert L.yskn_kvx_attn_post(ctypes.byref(bad), None) == -1 and b"null buffer" in L.yskn_kv4_last_error()
