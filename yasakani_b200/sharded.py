"""Sequence-sharded long-context decode: one process per GPU, one exchange per step.

The packed cache of one sequence is cut into contiguous token ranges, one per rank, on multiples of 32
tokens so that no K group straddles two ranks; the open fp16-shadow group lives on the last rank.  Every
rank runs the same split-K decode on its range, folds its partials into one (m, l, O) triple per head
(Hq*(HD+2) floats), the triples are all-gathered (NCCL over NVLink on GPUs, gloo in CPU tests) and every
rank merges them with the arithmetic of the single-GPU split merge.  The reference has no multi-GPU path
(README.md:37); the 1-GPU result is the oracle.

Two forms of the exchange: the NCCL all-gather (`exchange="nccl"`), and direct peer stores (`exchange="p2p"`): the
kernel that folds a shard's partials writes the triple into every rank's exchange buffer over NVLink and raises an
arrival counter there, waits for the other ranks' counters and merges (one launch; two launches when the grid is too
large to be resident as a whole).  The peer buffers are torch symmetric memory (plain
peer mappings; NVLink multicast is switched off) and NCCL is used only to set them up.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    """Global tokens [start, start+capacity) live on `rank`; only the last rank receives appended tokens."""
    world: int
    rank: int
    start: int
    capacity: int

    @property
    def is_last(self) -> bool:
        return self.rank == self.world - 1

    def local_rows(self, lo: int, hi: int):
        """Intersection of global rows [lo, hi) with this shard as (global_lo, global_hi), possibly empty."""
        a, b = max(lo, self.start), min(hi, self.start + self.capacity)
        return (a, b) if b > a else (a, a)


def plan_shards(ctx: int, world: int, rank: int, max_ctx: int | None = None) -> ShardPlan:
    """Split `ctx` cached tokens contiguously over `world` ranks on 32-token boundaries.

    Ranks 0..world-2 hold `per` tokens each (per a multiple of 32, ceil(ctx/world) rounded up); the last rank
    holds the remainder and has room up to `max_ctx` (a multiple of 64) for tokens appended later."""
    if world < 1 or not (0 <= rank < world) or ctx < 0:
        raise ValueError("bad shard request")
    max_ctx = max_ctx if max_ctx is not None else ((ctx + 64 + 63) // 64) * 64
    per = (((ctx + world - 1) // world) + 63) // 64 * 64 if world > 1 else max_ctx
    start = min(rank * per, (max_ctx // 64) * 64)
    if rank == world - 1:
        cap = max(64, max_ctx - start)
    else:
        cap = per
    return ShardPlan(world, rank, start, (cap + 63) // 64 * 64)


def gather_triples(mine: torch.Tensor, gathered: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather one (m, l, O) triple block per rank into `gathered` [world, *mine.shape].  The only collective."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        gathered[0].copy_(mine)
        return gathered
    # concatenated form (world*M rows): accepted by both the nccl and the gloo backend
    dist.all_gather_into_tensor(gathered.view(-1, *mine.shape[1:]), mine, group=group)
    return gathered


class ShardedDecoder:
    """Decode attention of ONE sequence whose KV4 cache is sharded over the ranks of `group`.

    All arithmetic runs in the CUDA library (kv4.launch_*); this class only owns buffers and the exchange."""

    def __init__(self, shape, plan: ShardPlan, splits: int, rope: torch.Tensor, M: int = 1, dtype=torch.float16, group=None,
                 exchange: str = "nccl", peer_exchange=None, early: bool = False):
        from . import kv4
        # early: positions and cached rows below them are final before the step's predecessor kernel ends (yskn_kv4_attn_ext)
        self.ext = kv4.attn_ext(early=True) if early else None
        self.kv4, self.shape, self.plan, self.splits, self.rope, self.M, self.group = kv4, shape, plan, splits, rope, M, group
        self.exchange, self.x = exchange, peer_exchange
        if exchange == "p2p" and peer_exchange is None:
            self._xbuf, self.x = make_peer_exchange(kv4, plan.world, plan.rank, M, shape.hq, shape.hd, group)
        self.layer = kv4.KvLayer(shape.hkv, shape.hd, plan.capacity)
        self.pm, self.pl, self.pacc = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
        self.mine = torch.empty((M, shape.hq, shape.hd + 2), dtype=torch.float32, device="cuda")
        self.gathered = torch.empty((plan.world, M, shape.hq, shape.hd + 2), dtype=torch.float32, device="cuda")
        self.o16 = torch.empty((M, shape.hq, shape.hd), dtype=dtype, device="cuda")
        self.d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")       # GLOBAL position of row 0
        self.d_lpos = torch.zeros(1, dtype=torch.int32, device="cuda")      # local position for appends

    def append(self, k_rows: torch.Tensor, v_rows: torch.Tensor, global_pos0: int) -> int:
        """Append the part of global rows [global_pos0, +n) that belongs to this shard; returns rows taken."""
        n = k_rows.shape[0]
        a, b = self.plan.local_rows(global_pos0, global_pos0 + n)
        if b <= a:
            return 0
        self.d_lpos.fill_(a - self.plan.start)
        self.kv4.launch_kv_append(self.layer, k_rows[a - global_pos0:b - global_pos0].contiguous(),
                                  v_rows[a - global_pos0:b - global_pos0].contiguous(), self.d_lpos, b - a)
        return b - a

    def local_step(self, q16: torch.Tensor) -> None:
        """Shard partials -> this rank's triple (enqueue only)."""
        s = self.shape
        self.kv4.launch_decode_shard_triple(q16, self.layer, self.M, self.d_pos, self.splits, self.pm, self.pl, self.pacc, self.rope,
                                            s.hq, s.qscale, s.rd, self.plan.start, self.plan.capacity, self.mine)

    def merge(self) -> torch.Tensor:
        s = self.shape
        self.kv4.launch_merge_triples(self.gathered, self.plan.world, self.M, s.hq, s.g, s.hd, self.o16)
        return self.o16

    def decode(self, q16: torch.Tensor) -> torch.Tensor:
        """q16 [M][Hq][HD] on this GPU (replicated on all ranks); self.d_pos must hold the global position."""
        s = self.shape
        if self.exchange == "p2p":
            self.kv4.launch_attention_shard(q16, self.layer, self.M, self.d_pos, self.splits, self.pm, self.pl, self.pacc, self.rope,
                                            s.hq, s.qscale, s.rd, self.plan.start, self.plan.capacity, ext=self.ext)
            if s.hq * self.M <= 148:                                 # one launch: fold, push, wait, merge
                self.kv4.launch_exchange_merge(self.pm, self.pl, self.pacc, self.splits, self.M, s.hq, s.g, s.hd, self.x, self.o16)
            else:
                self.kv4.launch_push_triple(self.pm, self.pl, self.pacc, self.splits, self.M, s.hq, s.hd, self.x)
                self.kv4.launch_merge_pushed(self.x, self.M, s.hq, s.g, s.hd, self.o16)
            return self.o16
        self.local_step(q16)
        gather_triples(self.mine, self.gathered, self.group)
        return self.merge()


def make_peer_exchange(kv4, world: int, rank: int, M: int, nh: int, hd: int, group=None):
    """Symmetric exchange buffer of every rank, zero-filled, and its descriptor.  Collective over `group`."""
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer mappings only
    import torch.distributed._symmetric_memory as symm
    n = kv4.exchange_bytes(world, M, nh, hd)
    buf = symm.empty((n + 3) // 4, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
    buf.zero_()
    hdl = symm.rendezvous(buf, group=group if group is not None else dist.group.WORLD)
    torch.cuda.synchronize()
    dist.barrier(group=group)                                          # nobody pushes into a buffer that is not cleared yet
    return (buf, hdl), kv4.peer_exchange(list(hdl.buffer_ptrs), rank)
