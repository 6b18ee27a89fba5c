"""Sequence-sharded decode on real GPUs: one process per GPU, both exchange forms, against the unsharded oracle.
Needs at least two GPUs; skipped otherwise (the shard plan, the exchange protocol and the merge are covered on one GPU
and on CPU by tests/test_gpu_attention.py and tests/test_sharded_cpu.py)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ctx, exchange, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import kv4_oracle as o
        from tests.helpers import f16_bits
        from yasakani_b200 import kv4, synth
        from yasakani_b200.sharded import ShardedDecoder, plan_shards
        shape = synth.C2
        k, v = synth.make_kv(shape, ctx + 1, seed=91)
        q = synth.make_q(shape, 1, seed=91)
        max_ctx = ((ctx + 128) // 64) * 64
        plan = plan_shards(ctx, world, rank, max_ctx)
        rope = torch.empty((max_ctx, shape.rd // 2, 2), dtype=torch.float32, device="cuda")
        kv4.launch_rope_table_g(rope, max_ctx, shape.theta, shape.rd)
        dec = ShardedDecoder(shape, plan, 9, rope, exchange=exchange)
        for p in range(0, ctx + 1, 1000):
            n = min(1000, ctx + 1 - p)
            dec.append(k[p:p + n].cuda(), v[p:p + n].cuda(), p)
        dec.d_pos.fill_(ctx)
        outs = []
        for _ in range(3):                                         # both halves of the exchange buffers
            outs.append(dec.decode(q.cuda()).float().cpu().numpy().copy())
        torch.cuda.synchronize()
        status = kv4.device_status()
        if rank == 0:
            okv = o.KvCache(shape.hkv, shape.hd, max_ctx)
            o.append(okv, 0, f16_bits(k), f16_bits(v))
            want = o.attention_exact(f16_bits(q), okv, ctx, o.rope_table(max_ctx, shape.theta, shape.rd), shape.hq, shape.rd, shape.qscale)
            err = max(float(np.max(np.abs(g - want) - 1e-2 * np.abs(want))) for g in outs)
            np.save(os.path.join(out_dir, "err.npy"), np.array([err, float(status)]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["p2p", "nccl"])
def test_sharded_decode_on_two_gpus(tmp_path, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), 5000, exchange, str(tmp_path)), nprocs=2, join=True)
    err, status = np.load(tmp_path / "err.npy")
    assert status == 0 and err <= 2e-3
