"""Host-side mirror of the reference's Family-A operator interface over the C ABI.

Function names and argument meaning follow the reference's launchers (src/args.hpp:14-21,
src/post_kernels.hpp:26,39-41); tensors are torch CUDA tensors used purely as device memory, and
every call is enqueue-only on torch's current stream.  All arithmetic happens in libyskn_kv4.so;
there is no torch or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from ._lib import F16, BF16, F32, KvLayerC, KvQuantArgsC, AttnGArgsC, AttnGCombineArgsC, KvAppendArgsC, PeerExchangeC, AttnExtC, MsRowsC, check

_NAMES = ("kq", "kscale", "kzero", "kshadow", "vq", "vscale", "vzero")


def _ptr(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device buffers must be contiguous CUDA tensors"
    return C.c_void_p(t.data_ptr())


def _stream(stream):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _dtype_code(t) -> int:
    if t.dtype in (torch.float16,):
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise TypeError(f"unsupported activation dtype {t.dtype}")


class KvLayer:
    """One layer's packed KV4 cache in the reference's layout (src/post_kernels.hpp:7-15), on one GPU."""

    def __init__(self, hkv: int, hd: int, max_ctx: int, device="cuda"):
        if max_ctx % 64 or hd not in (64, 128, 256):
            raise ValueError("max_ctx must be a multiple of 64 and head_dim one of 64/128/256")
        self.hkv, self.hd, self.max_ctx, self.device = hkv, hd, max_ctx, torch.device(device)
        ng = max_ctx // 32
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=self.device)
        self.kq = z((hkv, ng, 32, hd // 2), torch.uint8)
        self.kscale = z((hkv, ng, hd), torch.float16)
        self.kzero = z((hkv, ng, hd), torch.float16)
        self.kshadow = z((hkv, max_ctx, hd), torch.float16)
        self.vq = z((hkv, max_ctx, hd // 2), torch.uint8)
        self.vscale = z((hkv, max_ctx), torch.float16)
        self.vzero = z((hkv, max_ctx), torch.float16)

    def struct(self) -> KvLayerC:
        return KvLayerC(*[t.data_ptr() for t in self.tensors()])

    def tensors(self):
        return [getattr(self, n) for n in _NAMES]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())

    def to_numpy(self) -> dict:
        """Raw bytes of each array (fp16 arrays as uint16 bit patterns), for bit-exact comparison."""
        out = {}
        for n in _NAMES:
            t = getattr(self, n).cpu()
            out[n] = t.view(torch.int16).numpy().view("uint16") if t.dtype == torch.float16 else t.numpy()
        return out

    def load_numpy(self, arrays: dict) -> "KvLayer":
        import numpy as np
        for n in _NAMES:
            dst = getattr(self, n)
            a = np.ascontiguousarray(arrays[n])
            src = torch.from_numpy(a.view(np.int16)).view(torch.float16) if dst.dtype == torch.float16 else torch.from_numpy(a)
            dst.copy_(src.reshape(dst.shape))
        return self


def build_info() -> str:
    return _lib.load().yskn_kv4_build_info().decode()


def set_algo(algo: int) -> None:
    check(_lib.load().yskn_kv4_set_algo(int(algo)), "yskn_kv4_set_algo")


def device_status() -> int:
    """Status word of the tensor-core decode kernel (0 = ok); reading it synchronises and clears it."""
    v = C.c_int(0)
    check(_lib.load().yskn_kv4_device_status(C.byref(v)), "yskn_kv4_device_status")
    return v.value


def launch_rope_table_g(out: torch.Tensor, max_ctx: int, theta: float, rd: int, stream=None) -> None:
    """(cos,sin) float pairs [max_ctx][rd/2]; reference: launch_rope_table_g (src/attention_gqa.cu:166)."""
    assert out.dtype == torch.float32 and out.numel() >= max_ctx * rd
    check(_lib.load().yskn_kv4_rope_table(_ptr(out), max_ctx, C.c_float(theta), rd, _stream(stream)), "yskn_kv4_rope_table")


def launch_kv_append(kv: KvLayer, k_in: torch.Tensor, v_in: torch.Tensor, d_pos: torch.Tensor, M: int, stream=None) -> None:
    """K/V branches of launch_qkv_post (src/post_kernels.cu:48-82) + launch_kv_group_quant_g."""
    assert k_in.shape == v_in.shape and k_in.dtype == v_in.dtype and k_in.numel() == M * kv.hkv * kv.hd
    a = KvAppendArgsC(k_in.data_ptr(), v_in.data_ptr(), _dtype_code(k_in), kv.struct(), d_pos.data_ptr(), M, kv.max_ctx, kv.hkv, kv.hd)
    assert k_in.is_cuda and k_in.is_contiguous() and v_in.is_contiguous() and d_pos.dtype == torch.int32
    check(_lib.load().yskn_kv4_append(C.byref(a), _stream(stream)), "yskn_kv4_append")


def launch_kv_group_quant_g(kv: KvLayer, d_pos: torch.Tensor, M: int, stream=None) -> None:
    """launch_kv_group_quant_g (src/attention_gqa.cu:182-187)."""
    a = KvQuantArgsC(kv.struct(), d_pos.data_ptr(), M, kv.max_ctx)
    check(_lib.load().yskn_kv4_group_quant(C.byref(a), kv.hkv, kv.hd, _stream(stream)), "yskn_kv4_group_quant")


def attn_scratch(M: int, splits: int, nh: int, hd: int, device="cuda"):
    """pm, pl [M][splits][nh] and pacc [M][splits][nh][hd], sized as the reference sizes them (src/engine.cpp:560-561)."""
    pm = torch.empty((M, splits, nh), dtype=torch.float32, device=device)
    pl = torch.empty((M, splits, nh), dtype=torch.float32, device=device)
    pacc = torch.empty((M, splits, nh, hd), dtype=torch.float32, device=device)
    return pm, pl, pacc


def _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale) -> AttnGArgsC:
    assert q16.is_cuda and q16.is_contiguous() and q16.numel() == M * nh * kv.hd
    assert pm.numel() >= M * splits * nh and pacc.numel() >= M * splits * nh * kv.hd and d_pos.dtype == torch.int32
    return AttnGArgsC(q16.data_ptr(), kv.struct(), kv.max_ctx, M, d_pos.data_ptr(), splits, pm.data_ptr(), pl.data_ptr(),
                      pacc.data_ptr(), rope.data_ptr() if rope is not None else None, kv.hkv, nh, qscale)


def attn_ext(early: bool = False, splits_short: int = 0, long_len: int = 0, wk=None) -> AttnExtC:
    """yskn_kv4_attn_ext: the extras of the 27B engine's argument set (src/q35.hpp:126-130,136); `wk` a uint8 device tensor."""
    return AttnExtC(1 if early else 0, splits_short, long_len, wk.data_ptr() if wk is not None else None)


def launch_attention_gqa(q16, kv: KvLayer, M: int, d_pos, splits: int, pm, pl, pacc, rope, nh: int, qscale: float,
                         rd: int, stream=None, ext: AttnExtC | None = None) -> None:
    """launch_attention_gqa (src/attention_gqa.cu:168-175): split-K partials for M rows."""
    a = _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale)
    if ext is not None:
        check(_lib.load().yskn_kv4_attention_ex(C.byref(a), C.byref(ext), nh // kv.hkv, kv.hd, rd, _dtype_code(q16), _stream(stream)), "yskn_kv4_attention_ex")
        return
    check(_lib.load().yskn_kv4_attention(C.byref(a), nh // kv.hkv, kv.hd, rd, _dtype_code(q16), _stream(stream)), "yskn_kv4_attention")


class MsSlots:
    """Sequences bound to the slots of a multi-request pass (yskn_kv4_ms_prepare): device tables of their cache arrays and
    tensor maps.  All layers must share kvh, head_dim and max_ctx."""

    def __init__(self, layers: list):
        kv0 = layers[0]
        assert all(l.hkv == kv0.hkv and l.hd == kv0.hd and l.max_ctx == kv0.max_ctx for l in layers)
        self.layers, self.n, self.hkv, self.hd, self.max_ctx = layers, len(layers), kv0.hkv, kv0.hd, kv0.max_ctx
        L = _lib.load()
        self.d_layers = torch.empty(self.n * C.sizeof(KvLayerC), dtype=torch.uint8, device="cuda")
        self.d_maps = torch.empty(int(L.yskn_kv4_ms_maps_bytes(self.n)) + 128, dtype=torch.uint8, device="cuda")
        self.maps_ptr = (self.d_maps.data_ptr() + 127) // 128 * 128
        host = (KvLayerC * self.n)(*[l.struct() for l in layers])
        check(L.yskn_kv4_ms_prepare(host, self.n, self.hkv, self.hd, self.max_ctx, self.d_layers.data_ptr(), self.maps_ptr, _stream(None)),
              "yskn_kv4_ms_prepare")


def launch_attention_ms(q16, slots: MsSlots, M: int, pos, slot, splits: int, pm, pl, pacc, rope, nh: int, qscale: float, rd: int,
                        stream=None) -> None:
    """Partials for M rows of several sequences in one launch (yskn_kv4_attention_ms): pos, slot int32 device tensors [M]."""
    assert pos.dtype == torch.int32 and slot.dtype == torch.int32 and pos.numel() >= M and slot.numel() >= M
    a = AttnGArgsC(q16.data_ptr(), KvLayerC(), slots.max_ctx, M, None, splits, pm.data_ptr(), pl.data_ptr(), pacc.data_ptr(),
                   rope.data_ptr() if rope is not None else None, slots.hkv, nh, qscale)
    ms = MsRowsC(pos.data_ptr(), slot.data_ptr(), slots.d_layers.data_ptr(), slots.maps_ptr, slots.n)
    check(_lib.load().yskn_kv4_attention_ms(C.byref(a), C.byref(ms), nh // slots.hkv, slots.hd, rd, _dtype_code(q16), _stream(stream)),
          "yskn_kv4_attention_ms")


def launch_attention_shard(q16, kv: KvLayer, M: int, d_pos, splits: int, pm, pl, pacc, rope, nh: int, qscale: float,
                           rd: int, shard_start: int, shard_len: int, stream=None, ext: AttnExtC | None = None) -> None:
    """Partials over a cache holding only global tokens [shard_start, shard_start+shard_len); d_pos stays global."""
    a = _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale)
    check(_lib.load().yskn_kv4_attention_shard_ex(C.byref(a), C.byref(ext) if ext is not None else None, nh // kv.hkv, kv.hd, rd, _dtype_code(q16),
                                                 shard_start, shard_len, _stream(stream)), "yskn_kv4_attention_shard")


def launch_decode(q16, kv: KvLayer, M: int, d_pos, splits: int, pm, pl, pacc, rope, nh: int, qscale: float, rd: int, o16,
                  bv=None, gate=None, stream=None, ext: AttnExtC | None = None) -> None:
    """launch_attention_gqa + the merge of launch_attn_combine_gqa_xform as one launch where the shape allows
    (src/attention_gqa.cu:168-181).  Calls on one device must not overlap."""
    a = _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale)
    g = nh // kv.hkv
    c = AttnGCombineArgsC(pm.data_ptr(), pl.data_ptr(), pacc.data_ptr(), splits, M, bv.data_ptr() if bv is not None else None,
                          o16.data_ptr(), gate.data_ptr() if gate is not None else None, nh, g)
    check(_lib.load().yskn_kv4_decode_ex(C.byref(a), C.byref(c), C.byref(ext) if ext is not None else None, g, kv.hd, rd, _dtype_code(q16),
                                        _stream(stream)), "yskn_kv4_decode")


def launch_decode_shard_triple(q16, kv: KvLayer, M: int, d_pos, splits: int, pm, pl, pacc, rope, nh: int, qscale: float, rd: int,
                               shard_start: int, shard_len: int, triple, stream=None) -> None:
    """Shard partials and their fold into this shard's (m, l, O) triple [M][nh][hd+2], one launch where the shape allows."""
    a = _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale)
    check(_lib.load().yskn_kv4_decode_shard_triple(C.byref(a), nh // kv.hkv, kv.hd, rd, _dtype_code(q16), shard_start, shard_len,
                                                  _ptr(triple), _stream(stream)), "yskn_kv4_decode_shard_triple")


def launch_attn_combine_gqa(pm, pl, pacc, splits: int, M: int, o16, nh: int, g: int, bv=None, gate=None, stream=None) -> None:
    """Merge half of launch_attn_combine_gqa_xform (src/attention_gqa.cu:123-134,176-181), up to the o16 store."""
    hd = o16.numel() // (M * nh)
    a = AttnGCombineArgsC(pm.data_ptr(), pl.data_ptr(), pacc.data_ptr(), splits, M, bv.data_ptr() if bv is not None else None,
                          o16.data_ptr(), gate.data_ptr() if gate is not None else None, nh, g)
    check(_lib.load().yskn_kv4_combine(C.byref(a), hd, _dtype_code(o16), _stream(stream)), "yskn_kv4_combine")


def launch_xform_a8(o16, signs, qx, alpha, stream=None) -> None:
    """Sign flip, Hadamard-512, int8 codes + fp32 scale per 512 values of the merged rows (yskn_kv4_xform_a8): o16 fp16 [M][nh][hd],
    signs int8 [nh*hd], qx int8 like o16, alpha fp32 [M][nh*hd/512]."""
    M = o16.shape[0]
    n = o16.numel() // M
    assert o16.dtype == torch.float16 and signs.dtype == torch.int8 and qx.dtype == torch.int8 and alpha.dtype == torch.float32
    check(_lib.load().yskn_kv4_xform_a8(_ptr(o16), _ptr(signs), _ptr(qx), _ptr(alpha), M, n, _stream(stream)), "yskn_kv4_xform_a8")


def launch_attention_prefill(q16, kv: KvLayer, M: int, d_pos, splits: int, pm, pl, pacc, rope, nh: int, qscale: float,
                             rd: int, o16, bv=None, stream=None) -> None:
    """launch_attention_prefill (src/attention_kv4q.cu:449-453): attention of M appended rows, merged to o16."""
    a = _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale)
    check(_lib.load().yskn_kv4_prefill(C.byref(a), nh // kv.hkv, kv.hd, rd, _dtype_code(q16), bv.data_ptr() if bv is not None else None,
                                      _ptr(o16), _stream(stream)), "yskn_kv4_prefill")


def set_tc_workspace(ws: torch.Tensor | None) -> None:
    """Lend (or, with None, take back) a workspace so that the plain attention entries use the tcgen05 kernel for passes of
    more than 8 rows on the current device (yskn_kv4_set_tc_workspace).  Keep the tensor alive while it is lent."""
    check(_lib.load().yskn_kv4_set_tc_workspace(ws.data_ptr() if ws is not None else None, ws.numel() * ws.element_size() if ws is not None else 0),
          "yskn_kv4_set_tc_workspace")


def tc_workspace(kv: KvLayer, M: int) -> torch.Tensor:
    """Caller-owned fp16 workspace of the tensor-core multi-row path (the reference's KvF32 arrays, src/args.hpp:37)."""
    n = _lib.load().yskn_kv4_tc_workspace_bytes(kv.hkv, kv.hd, kv.max_ctx, M)
    if n == 0:
        raise ValueError("unsupported shape for the tensor-core path")
    return torch.empty(n, dtype=torch.uint8, device=kv.device)


def launch_attention_tc(q16, kv: KvLayer, M: int, d_pos, splits: int, pm, pl, pacc, rope, nh: int, qscale: float, rd: int,
                        workspace: torch.Tensor | None, valid_tokens: int = 0, stream=None) -> None:
    """launch_kv_dequant + launch_attention_f32 (src/attention_kv4q.cu:198-285) on tcgen05: partials for M rows.
    workspace None: the kernel converts the packed cache itself (no dequantised copy, one launch)."""
    a = _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale)
    check(_lib.load().yskn_kv4_attention_tc(C.byref(a), nh // kv.hkv, kv.hd, rd, _dtype_code(q16), _ptr(workspace) if workspace is not None else None,
                                           workspace.numel() if workspace is not None else 0, valid_tokens, _stream(stream)), "yskn_kv4_attention_tc")


def launch_attention_prefill_tc(q16, kv: KvLayer, M: int, d_pos, splits: int, pm, pl, pacc, rope, nh: int, qscale: float, rd: int,
                                o16, workspace: torch.Tensor | None, bv=None, valid_tokens: int = 0, stream=None) -> None:
    """launch_attention_prefill_f32 (src/attention_kv4q.cu:287-323) on tcgen05: M appended rows, merged to o16.
    workspace None: the kernel converts the packed cache itself."""
    a = _attn_args(q16, kv, M, d_pos, splits, pm, pl, pacc, rope, nh, qscale)
    check(_lib.load().yskn_kv4_prefill_tc(C.byref(a), nh // kv.hkv, kv.hd, rd, _dtype_code(q16), bv.data_ptr() if bv is not None else None,
                                         _ptr(o16), _ptr(workspace) if workspace is not None else None,
                                         workspace.numel() if workspace is not None else 0, valid_tokens, _stream(stream)), "yskn_kv4_prefill_tc")


def launch_local_triple(pm, pl, pacc, splits: int, M: int, nh: int, hd: int, triple, stream=None) -> None:
    """Fold one shard's partials into (m, l, O) per (row, head): float [M][nh][hd+2]."""
    a = AttnGCombineArgsC(pm.data_ptr(), pl.data_ptr(), pacc.data_ptr(), splits, M, None, None, None, nh, 1)
    check(_lib.load().yskn_kv4_local_triple(C.byref(a), hd, _ptr(triple), _stream(stream)), "yskn_kv4_local_triple")


def launch_merge_triples(triples, ranks: int, M: int, nh: int, g: int, hd: int, o16, bv=None, gate=None, stream=None) -> None:
    """Merge triples gathered from all shards, [ranks][M][nh][hd+2], into o16."""
    check(_lib.load().yskn_kv4_merge_triples(_ptr(triples), ranks, M, nh, g, hd, bv.data_ptr() if bv is not None else None,
                                            gate.data_ptr() if gate is not None else None, _ptr(o16), _dtype_code(o16),
                                            _stream(stream)), "yskn_kv4_merge_triples")


def decode_noalloc(q16, kv: KvLayer, d_pos, splits: int, rope, nh: int, qscale: float, rd: int, o16, stream=None) -> None:
    """One decode step with the split-K scratch held inside the library (no buffer to allocate); M = 1 and
    splits * nh * (hd + 2) <= 528,384 floats.  Calls on one GPU share that scratch and must not overlap."""
    s = kv.struct()
    check(_lib.load().yskn_kv4_decode_noalloc(_ptr(q16), C.byref(s), kv.max_ctx, _ptr(d_pos), splits, rope.data_ptr() if rope is not None else None,
                                             kv.hkv, nh, kv.hd, rd, C.c_float(qscale), _dtype_code(q16), _ptr(o16), _stream(stream)),
          "yskn_kv4_decode_noalloc")


def set_peer_wait_polls(polls: int) -> None:
    """Limit of the wait for the other shards' triples in poll rounds of ~0.5 us; 0 restores the default (yskn_kv4_set_peer_wait_polls)."""
    check(_lib.load().yskn_kv4_set_peer_wait_polls(int(polls)), "yskn_kv4_set_peer_wait_polls")


def exchange_bytes(world: int, M: int, nh: int, hd: int) -> int:
    return int(_lib.load().yskn_kv4_exchange_bytes(world, M, nh, hd))


def peer_exchange(buffer_ptrs, rank: int) -> PeerExchangeC:
    """Descriptor of the ranks' exchange buffers as mapped into this process (buffer_ptrs[rank] is the local one)."""
    x = PeerExchangeC()
    for w, p in enumerate(buffer_ptrs):
        x.buf[w] = int(p)
    x.world, x.rank = len(buffer_ptrs), rank
    return x


def launch_push_triple(pm, pl, pacc, splits: int, M: int, nh: int, hd: int, x: PeerExchangeC, stream=None) -> None:
    """Fold this shard's partials into its (m, l, O) triple and store it into every rank's exchange buffer (peer stores)."""
    a = AttnGCombineArgsC(pm.data_ptr(), pl.data_ptr(), pacc.data_ptr(), splits, M, None, None, None, nh, 1)
    check(_lib.load().yskn_kv4_push_triple(C.byref(a), hd, C.byref(x), _stream(stream)), "yskn_kv4_push_triple")


def launch_merge_pushed(x: PeerExchangeC, M: int, nh: int, g: int, hd: int, o16, bv=None, gate=None, stream=None) -> None:
    """Wait (bounded) for every rank's pushed triple of this step and merge them into o16."""
    check(_lib.load().yskn_kv4_merge_pushed(C.byref(x), M, nh, g, hd, bv.data_ptr() if bv is not None else None,
                                           gate.data_ptr() if gate is not None else None, _ptr(o16), _dtype_code(o16), _stream(stream)),
          "yskn_kv4_merge_pushed")


def launch_exchange_merge(pm, pl, pacc, splits: int, M: int, nh: int, g: int, hd: int, x: PeerExchangeC, o16, bv=None, gate=None, stream=None) -> None:
    """Push and merge in one launch (nh * M <= 148): fold, store to all ranks, wait for theirs, merge into o16."""
    a = AttnGCombineArgsC(pm.data_ptr(), pl.data_ptr(), pacc.data_ptr(), splits, M, bv.data_ptr() if bv is not None else None, o16.data_ptr(),
                          gate.data_ptr() if gate is not None else None, nh, g)
    check(_lib.load().yskn_kv4_exchange_merge(C.byref(a), hd, _dtype_code(o16), C.byref(x), _stream(stream)), "yskn_kv4_exchange_merge")


def default_qscale(hd: int) -> float:
    return 1.0 / math.sqrt(hd)


def copy_small(dst: torch.Tensor, src: torch.Tensor, stream=None) -> None:
    """yskn_kv4_copy: dst <- src by a kernel; either tensor may live in pinned host memory.  Sizes and addresses multiples of 16."""
    nbytes = src.numel() * src.element_size()
    if nbytes != dst.numel() * dst.element_size() or not (src.is_contiguous() and dst.is_contiguous()):
        raise ValueError("copy_small: contiguous tensors of equal size")
    for t in (dst, src):
        if not (t.is_cuda or t.is_pinned()):
            raise ValueError("copy_small: host tensors must be pinned")
    check(_lib.load().yskn_kv4_copy(dst.data_ptr(), src.data_ptr(), nbytes, _stream(stream)), "yskn_kv4_copy")
