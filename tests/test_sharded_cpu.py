"""Host logic of the sequence-sharded decode on CPU: shard plan, the one exchange (gloo, world_size 2 and 3),
and the triple merge, with the oracle standing in for the per-shard CUDA kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from yasakani_b200 import synth
from yasakani_b200.sharded import gather_triples, plan_shards


@pytest.mark.parametrize("ctx,world", [(262144, 1), (262144, 2), (262144, 8), (1000, 4), (31, 2), (4096, 3)])
def test_plan_covers_every_token_once_on_group_boundaries(ctx, world):
    plans = [plan_shards(ctx, world, r) for r in range(world)]
    assert plans[0].start == 0
    for a, b in zip(plans, plans[1:]):
        assert a.start + a.capacity == b.start or b.start >= ctx or a.start + a.capacity >= b.start
        assert b.start % 32 == 0
    for p in plans:
        assert p.capacity % 64 == 0 and p.start % 32 == 0
    # every cached token and the next appended token fall in exactly one shard
    for t in list(range(0, ctx + 1, max(1, ctx // 97))) + [ctx]:
        owners = [p.rank for p in plans if p.start <= t < p.start + p.capacity]
        assert len(owners) == 1, (t, owners)
    assert plans[-1].is_last and plans[-1].start + plans[-1].capacity > ctx


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ctx, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import kv4_oracle as o
        from tests.helpers import f16_bits
        shape = synth.Shape(12, 2, 128, 64, 1e6)
        k, v = synth.make_kv(shape, ctx + 1, seed=77)
        q16 = f16_bits(synth.make_q(shape, 1, seed=77))
        k16, v16 = f16_bits(k), f16_bits(v)
        plan = plan_shards(ctx, world, rank)
        rope = o.rope_table(((ctx + 128) // 64) * 64, shape.theta, shape.rd)
        # this rank's shard: the same append calls a GPU rank makes, on local positions
        kv = o.KvCache(shape.hkv, shape.hd, plan.capacity)
        a, b = plan.local_rows(0, ctx + 1)
        if b > a:
            o.append(kv, a - plan.start, k16[a:b], v16[a:b])
        pm, pl, pacc = o.attention_partials(q16, kv, ctx, 4, rope, shape.hq, shape.rd, shape.qscale, threads=1,
                                            shard_start=plan.start, shard_len=plan.capacity)
        # fold the 4 local splits into one triple (what yskn_kv4_local_triple does)
        M2 = pm[0].max(0); w = np.where(pm[0] > -1e29, np.exp(pm[0] - M2), 0.0)
        mine = np.concatenate([M2[:, None], (w * pl[0]).sum(0)[:, None], (w[..., None] * pacc[0]).sum(0)], -1).astype(np.float32)
        mine_t = torch.from_numpy(mine)[None]                                      # [M=1][hq][hd+2]
        gathered = torch.empty((world,) + tuple(mine_t.shape), dtype=torch.float32)
        gather_triples(mine_t, gathered)
        merged = o.merge_triples(gathered[:, 0].numpy())
        # oracle of the sharded path: the unsharded result
        full = o.KvCache(shape.hkv, shape.hd, ((ctx + 128) // 64) * 64)
        o.append(full, 0, k16, v16)
        want = o.attention_exact(q16, full, ctx, rope, shape.hq, shape.rd, shape.qscale, threads=1)[0]
        np.save(os.path.join(out_dir, f"err{rank}.npy"), np.abs(merged - want).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,ctx", [(2, 517), (3, 95), (2, 20)])
def test_sharded_merge_equals_unsharded_result_gloo(tmp_path, world, ctx):
    mp.spawn(_worker, args=(world, _free_port(), ctx, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")) < 2e-5
