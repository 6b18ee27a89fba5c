#!/usr/bin/env python
"""Benchmark of the KV4 decode-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--ctx 262144]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one decode step of one full-attention layer for one sequence: split-K attention of one query token
(Hq 24 / Hkv 4 / head_dim 256) over a KV4 cache of `ctx` tokens, then the split merge to o16.  With N > 1
the cache is sequence-sharded over the ranks and the step adds the one (m, l, O) all-gather (strong scaling:
the total work is fixed).  Inputs are seeded synthetic rows (yasakani_b200/synth.py), quantised by the
library's own codec.  Rank 0 prints one JSON line.

--impl reference times the CPU restatement of the reference's algorithm (oracle/, test infrastructure) on the
host cores: the reference has no CPU implementation of this path and its CUDA kernels are not a CPU arm.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from yasakani_b200 import synth  # noqa: E402

CONFIG_INDEX = 3                    # BASELINE.json configs[3]: long-context single-sequence decode, 262,144 tokens
CHUNK = 8192                        # rows generated, uploaded and appended per pass
METRIC, UNIT = "kv4_decode_attn_tokens_per_s", "tokens/s"


def chunk_rows(shape, c):
    """Rows of global tokens [c*CHUNK, (c+1)*CHUNK): the same on every rank and in the CPU arm."""
    return synth.make_kv(shape, CHUNK, synth.seed_for(CONFIG_INDEX, c))


def workload_name(shape, ctx):
    return f"C4 long-context decode: 1 query token, Hq{shape.hq}/Hkv{shape.hkv}/hd{shape.hd}, KV4 cache of {ctx} tokens"


def bench_config(shape, ctx, world):
    """What is measured; printed identically by both arms (how our arm runs it is under `run`)."""
    return {"workload": workload_name(shape, ctx), "context_tokens": ctx, "parallelism": f"sequence-sharded x{world}",
            "l2": "inputs larger than L2: consecutive launches read different cache copies, at least 256 MB per cycle (L2 is 126 MB)"}


def host_threads():
    """Threads for the CPU arm: the cores this process may run on.  torch.distributed.run exports OMP_NUM_THREADS=1,
    which would otherwise hold the OpenMP oracle to one thread."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


# ------------------------------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True); self.t.start()
        except OSError:
            self.proc = None
        return self

    def wait_started(self, timeout_s: float = 1.5):
        t0 = time.time()
        while self.proc is not None and not self.rows and time.time() - t0 < timeout_s:
            time.sleep(0.01)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ CPU arm

def cpu_decode_rate(shape, ctx, sample_ctx, steps, warmup, threads, kv=None):
    """Times the oracle's reference-literal decode (split-K partials + merge) over the first `sample_ctx` tokens of a cache
    and scales the step time by ctx/sample_ctx (the work is linear in the number of keys).  `kv`: a cache that already
    holds at least `sample_ctx` tokens; built with the oracle's codec otherwise."""
    from oracle import kv4_oracle as o
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if kv is None:
        kv = o.KvCache(shape.hkv, shape.hd, ((sample_ctx + 63) // 64) * 64)
        for c in range((sample_ctx + CHUNK - 1) // CHUNK):
            k, v = chunk_rows(shape, c)
            n = min(CHUNK, sample_ctx - c * CHUNK)
            o.append(kv, c * CHUNK, bits(k[:n]), bits(v[:n]))
    max_ctx = kv.max_ctx
    rope = o.rope_table(max_ctx, shape.theta, shape.rd)
    q16 = bits(synth.make_q(shape, 1, synth.seed_for(CONFIG_INDEX)))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        pm, pl, pacc = o.attention_partials(q16, kv, sample_ctx - 1, 32, rope, shape.hq, shape.rd, shape.qscale, threads=threads)
        o16 = o.combine(pm, pl, pacc, shape.g)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    step_s = float(np.mean(times)) * (ctx / sample_ctx)
    return step_s, o16, (kv, rope, q16)


def run_reference(args, rank, world):
    """The reference arm: the CPU restatement on all host threads; rank 0 only."""
    if rank != 0:
        return
    from oracle import kv4_oracle as o
    shape, ctx = synth.C2, args.ctx
    threads = host_threads()
    budget = max(0.05, min(2.0, 100.0 / (args.steps + args.warmup)))          # seconds of CPU work per step
    probe_s, _, _ = cpu_decode_rate(shape, 4096, 4096, 1, 1, threads)         # seconds per step at 4,096 keys
    sample_ctx = int(min(ctx, max(4096, (budget / probe_s * 4096) // 4096 * 4096)))
    step_s, _, _ = cpu_decode_rate(shape, ctx, sample_ctx, args.steps, args.warmup, threads)
    value = 1.0 / step_s
    sample = f"each step = reference-literal decode over the first {sample_ctx} of {ctx} keys, time scaled by {ctx / sample_ctx:.1f}"
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "impl": "reference", "config": bench_config(shape, ctx, world),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ our arm

def peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from yasakani_b200 import kv4
    from yasakani_b200.sharded import ShardedDecoder, gather_triples, plan_shards

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path for the product arm"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    shape, ctx, K, W = synth.C2, args.ctx, args.steps, args.warmup
    max_ctx = ctx + 64
    plan = plan_shards(ctx, world, rank, max_ctx)
    splits = args.splits

    rope = torch.empty((max_ctx, shape.rd // 2, 2), dtype=torch.float32, device=dev)
    kv4.launch_rope_table_g(rope, max_ctx, shape.theta, shape.rd)

    # ---- build this rank's shard with the library's own codec, then clone it so timed loops miss L2
    exchange = args.exchange if world > 1 else "nccl"
    xch = None
    if exchange == "p2p":
        from yasakani_b200.sharded import make_peer_exchange
        try:
            xkeep, xch = make_peer_exchange(kv4, world, rank, 1, shape.hq, shape.hd)
        except Exception as e:                                      # symmetric memory unavailable: the NCCL form still works
            if rank == 0:
                print(f"[bench] peer exchange unavailable ({type(e).__name__}: {e}); using the NCCL all-gather", file=sys.stderr)
            exchange = "nccl"
    # `early`: in this workload the position and every cached row below it are final long before a step starts (the appended
    # row sits AT the position), which is what the flag promises; the decode kernel then fills its ring ahead of the wait
    early = not args.no_early
    ext = kv4.attn_ext(early=True) if early else None
    first = ShardedDecoder(shape, plan, splits, rope, exchange=exchange, peer_exchange=xch, early=early)
    lo, hi = plan.local_rows(0, ctx)
    for c in range(lo // CHUNK, (hi + CHUNK - 1) // CHUNK if hi > lo else 0):
        k, v = chunk_rows(shape, c)
        first.append(k.to(dev), v.to(dev), c * CHUNK)
    torch.cuda.synchronize()
    shard_tokens = hi - lo
    shard_bytes = shape.decode_bytes(shard_tokens)                 # algorithmic bytes one launch of the decode kernel reads
    n_copies = max(2, int(math.ceil(256e6 / max(shard_bytes, 1))) + 1)
    decs = [first]
    for _ in range(n_copies - 1):
        d = ShardedDecoder(shape, plan, splits, rope, exchange=exchange, peer_exchange=xch, early=early)
        for a, b in zip(d.layer.tensors(), first.layer.tensors()):
            a.copy_(b)
        decs.append(d)
    for d in decs:
        d.d_pos.fill_(ctx - 1)                                      # the query is the last cached token: ctx keys visible
    # one staging buffer per side for a step's inputs: the query row and the new token's K and V rows, so that the
    # end-to-end step moves them with a single host-to-device copy
    nq, nkv = shape.hq * shape.hd, shape.hkv * shape.hd
    in_host = torch.empty(nq + 2 * nkv, dtype=torch.float16).pin_memory()
    in_dev = torch.empty(nq + 2 * nkv, dtype=torch.float16, device=dev)
    q_host = in_host[:nq].view(1, shape.hq, shape.hd)
    q_host.copy_(synth.make_q(shape, 1, synth.seed_for(CONFIG_INDEX)))
    q_dev = in_dev[:nq].view(1, shape.hq, shape.hd)
    q_dev.copy_(q_host)
    o_host = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16).pin_memory()

    def step(d):
        if world > 1:
            d.decode(q_dev)
        else:
            kv4.launch_decode(q_dev, d.layer, 1, d.d_pos, splits, d.pm, d.pl, d.pacc, rope, shape.hq, shape.qscale, shape.rd, d.o16, ext=ext)

    # attention + merge (N = 1); attention + fused push/wait/merge (N > 1, p2p); attention + triple + merge of triples (N > 1, nccl)
    launches_per_step = 3 if (world > 1 and exchange == "nccl") else 2

    # CUDA graphs: the step is launch-bound otherwise (a few 10 us of kernels).  One graph per cache copy holds one step (used
    # by the end-to-end loop, which copies host buffers between steps); one more holds GSTEPS consecutive steps over the
    # copies in turn, the way a decode pass runs the attention of all its layers inside one captured graph (the reference
    # captures whole passes, src/engine35.cpp:1973-1989): a graph launch costs about 5 us, a kernel node inside one about 2.
    side = torch.cuda.Stream(device=dev)
    graphs = []
    with torch.cuda.stream(side):
        for d in decs:
            step(d)                                                # warm up outside capture (module load, NCCL setup)
        torch.cuda.synchronize()
        for d in decs:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                step(d)
            graphs.append(g)
        pass_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(pass_graph, stream=side):
            for s_ in range(GSTEPS):
                step(decs[s_ % n_copies])
    torch.cuda.synchronize()

    def run_steps(n):                                              # exactly n steps: whole passes, then single steps
        for _ in range(n // GSTEPS):
            pass_graph.replay()
        for i in range(n % GSTEPS):
            graphs[i % n_copies].replay()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = ClockSampler(local_rank)
    with sampler:
        # ---- value: inputs resident in HBM, whole step (attention + merge [+ exchange])
        sampler.wait_started()                                     # nvidia-smi takes ~0.1 s to deliver its first sample
        timed(lambda i: run_steps(W), 1)
        # exactly K steps per measurement; short runs are measured several times (median reported, the same number of times
        # on every rank) so that the clock samples, 20 ms apart, fall inside timed regions
        probe = timed(lambda i: run_steps(K), 1)
        reps = int(min(7, max(1, math.ceil(150.0 / max(probe, 1e-3))))) | 1
        ms_total = float(np.median([probe] + [timed(lambda i: run_steps(K), 1) for _ in range(reps - 1)]))
        # ---- roofline: the decode-attention kernel alone, same stream, same copies, GSTEPS launches per captured graph so that
        #      the figure is a kernel time and not the host's launch rate (short shards run faster than ctypes can launch)
        def attn_only(d):
            kv4.launch_attention_shard(q_dev, d.layer, 1, d.d_pos, splits, d.pm, d.pl, d.pacc, rope, shape.hq, shape.qscale, shape.rd,
                                       plan.start, plan.capacity, ext=ext)
        with torch.cuda.stream(side):
            attn_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(attn_graph, stream=side):
                for s_ in range(GSTEPS):
                    attn_only(decs[s_ % n_copies])
        torch.cuda.synchronize()
        attn_replays = max(1, (K + GSTEPS - 1) // GSTEPS)
        timed(lambda i: attn_graph.replay(), max(1, W // GSTEPS))
        ms_attn = timed(lambda i: attn_graph.replay(), attn_replays)
        attn_launches = attn_replays * GSTEPS
        # ---- e2e: host buffers in, host buffer out, every step (q, and the new token's k/v on the owning rank)
        k_new, v_new = chunk_rows(shape, (ctx - 1) // CHUNK)
        kn_host = in_host[nq:nq + nkv].view(1, shape.hkv, shape.hd); vn_host = in_host[nq + nkv:].view(1, shape.hkv, shape.hd)
        kn_host.copy_(k_new[(ctx - 1) % CHUNK:(ctx - 1) % CHUNK + 1]); vn_host.copy_(v_new[(ctx - 1) % CHUNK:(ctx - 1) % CHUNK + 1])
        kn_dev = in_dev[nq:nq + nkv].view(1, shape.hkv, shape.hd); vn_dev = in_dev[nq + nkv:].view(1, shape.hkv, shape.hd)
        for d in decs:                                             # the new token's local position: constant over the run
            d.d_lpos.fill_(ctx - 1 - plan.start)

        def e2e_body(d):                                           # host buffers in, the step, host buffer out
            # the copies to and from pinned host memory: by the library's copy kernel (yskn_kv4_copy), or as memcpy nodes
            if args.e2e_copies == "kernel":
                kv4.copy_small(in_dev, in_host)
            else:
                in_dev.copy_(in_host, non_blocking=True)
            if plan.is_last:
                kv4.launch_kv_append(d.layer, kn_dev, vn_dev, d.d_lpos, 1)
            step(d)
            if rank == 0:
                if args.e2e_copies == "kernel":
                    kv4.copy_small(o_host, d.o16)
                else:
                    o_host.copy_(d.o16, non_blocking=True)

        # the whole step, copies included, is one captured graph per cache copy (the copies become memcpy nodes that run on
        # every replay); the host waits for the result after each step, as a caller that samples the next token would
        e2e_graphs = []
        with torch.cuda.stream(side):
            for d in decs:
                e2e_body(d)
            torch.cuda.synchronize()
            for d in decs:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    e2e_body(d)
                e2e_graphs.append(g)
        torch.cuda.synchronize()

        def e2e_step(i):
            e2e_graphs[i % n_copies].replay()
            torch.cuda.current_stream().synchronize()               # the caller consumes o16 on the host

        with torch.cuda.stream(side):
            timed(e2e_step, W)
            ms_e2e = timed(e2e_step, K)
    clocks = sampler.summary()

    peak, peak_kind = peak_hbm()
    t_attn = ms_attn / attn_launches * 1e-3
    achieved = shard_bytes / t_attn / 1e9
    value = K / (ms_total * 1e-3)
    # DRAM bytes of one decode-kernel launch: dram__bytes_read.sum + dram__bytes_write.sum from an ncu capture of this
    # bench at 262,144 tokens on one GPU (308.47 MB read, 0.1-3.5 MB written: 1.013 x the algorithmic bytes); for a
    # shard the figure scales with the tokens it holds.  --traffic overrides it with a fresh capture.
    traffic = args.traffic if args.traffic is not None else NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * shard_bytes
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": bench_config(shape, ctx, world),
        "run": {"splits": splits, "early_prefetch": early, "graph": f"{GSTEPS} steps (layers) per CUDA graph replay", "exchange": exchange if world > 1 else None,
                "cache_copies": n_copies, "mb_read_per_launch": shard_bytes / 1e6, "kv_tokens_scanned_per_s": ctx * value},
        "clocks": clocks,
        "e2e": {"value": K / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(q_host.numel() * 2 + (kn_host.numel() + vn_host.numel()) * 2),
                "d2h_bytes_per_step": int(o_host.numel() * 2), "ms_per_step": ms_e2e / K,
                "copies": "yskn_kv4_copy kernel nodes from / to pinned host memory" if args.e2e_copies == "kernel" else "cudaMemcpyAsync nodes from / to pinned host memory"},
        "gpu_launches": launches_per_step * K,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                     "kernel": "decode attention (split-K partials)", "us_per_launch": t_attn * 1e6, "bytes_per_launch": shard_bytes,
                     "peak_kind": f"of {peak_kind}", "timing": f"CUDA events around graph replays of {GSTEPS} launches over the cache copies"},
    }

    # ---- result check at every N: one more step at the full context on every rank; rank 0 compares the (sharded) o16 with the
    #      exact oracle over ALL `ctx` keys of the same packed cache and, for N > 1, with the 1-GPU decode of the unsharded
    #      cache; every rank's device status word (bounded waits that ran out) is reduced with MAX.
    from oracle import kv4_oracle as o
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    d = decs[0]
    d.d_pos.fill_(ctx - 1)
    step(d)
    torch.cuda.synchronize()
    st = torch.tensor([kv4.device_status()], dtype=torch.int32, device=dev)
    if world > 1:
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
    status = int(st.item())
    ok = True
    if rank == 0:
        got = d.o16.float().cpu().numpy()
        check = {"device_status_max_over_ranks": status}
        if world == 1:
            full = first.layer
        else:                                                       # the unsharded cache on rank 0's GPU, built by the same codec
            full = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
            fpos = torch.zeros(1, dtype=torch.int32, device=dev)
            for c in range((ctx + CHUNK - 1) // CHUNK):
                k, v = chunk_rows(shape, c)
                n = min(CHUNK, ctx - c * CHUNK)
                fpos.fill_(c * CHUNK)
                kv4.launch_kv_append(full, k[:n].to(dev), v[:n].to(dev), fpos, n)
            fpos.fill_(ctx - 1)
            pm1, pl1, pacc1 = kv4.attn_scratch(1, splits, shape.hq, shape.hd)
            o1 = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16, device=dev)
            kv4.launch_decode(q_dev, full, 1, fpos, splits, pm1, pl1, pacc1, rope, shape.hq, shape.qscale, shape.rd, o1)
            torch.cuda.synchronize()
            one = o1.float().cpu().numpy()
            e1 = np.abs(got - one)
            check["max_abs_diff_vs_1gpu"] = float(e1.max())
            check["ok_vs_1gpu"] = bool((e1 <= 2e-3 + 1e-2 * np.abs(one)).all())
        okv = o.KvCache(shape.hkv, shape.hd, max_ctx)
        for name, arr in full.to_numpy().items():
            getattr(okv, name)[...] = arr.reshape(getattr(okv, name).shape)
        # the packed cache itself: the first chunk re-encoded by the oracle's codec must give the same bytes
        ochk = o.KvCache(shape.hkv, shape.hd, CHUNK)
        k0, v0 = chunk_rows(shape, 0)
        o.append(ochk, 0, bits(k0), bits(v0))
        check["codec_first_chunk_bit_exact"] = bool(all(np.array_equal(getattr(ochk, nm)[:, :a], getattr(okv, nm)[:, :a])
                                                        for nm, a in (("kq", CHUNK // 32), ("kscale", CHUNK // 32), ("kzero", CHUNK // 32),
                                                                      ("vq", CHUNK), ("vscale", CHUNK), ("vzero", CHUNK))))
        threads = host_threads()
        want = o.attention_exact(bits(q_host), okv, ctx - 1, rope.cpu().numpy(), shape.hq, shape.rd, shape.qscale, threads=threads)
        err = np.abs(got - want)
        check.update({"keys": ctx, "max_abs_err_vs_oracle": float(err.max()), "ok_vs_oracle": bool((err <= 2e-3 + 1e-2 * np.abs(want)).all())})
        ok = bool(check["ok_vs_oracle"] and check.get("ok_vs_1gpu", True) and check["codec_first_chunk_bit_exact"] and status == 0)
        check["ok"] = ok
        line["check"] = check
        # ---- CPU baseline beside it (N = 1 only): the oracle's reference-literal decode on the host cores, bounded sample
        if world == 1 and not args.no_cpu_baseline:
            sample_ctx = min(ctx, args.cpu_sample_ctx)
            step_s, _, _ = cpu_decode_rate(shape, ctx, sample_ctx, 3, 1, threads, kv=okv)
            line["cpu_baseline"] = {"value": 1.0 / step_s, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"3 reference-literal decode steps over the first {sample_ctx} of {ctx} keys, time scaled by {ctx / sample_ctx:.1f}"}
        del okv, full
        if world == 1 and not args.no_secondary:
            del decs[1:]
            torch.cuda.empty_cache()
            line["secondary"] = secondary_lines(shape, splits, dev)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
    if not ok:
        sys.exit(3)


NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 310.27e6 / 306208768
GSTEPS = 16                                                        # steps per captured pass: the reference model has 16 attention layers


# ---------------------------------------------------------------------------------------------------------------
# Secondary workloads (--workload): the other kernels of the path, one GPU, device-timed, one JSON line each.
# They are not the headline metric; they make the numbers quoted for these kernels reproducible from this file.
def _timed(fn, steps, warmup):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1e-3


def _timed_graph(fn, steps, warmup, per_graph=8):
    """Like _timed, but the calls are captured into a CUDA graph of `per_graph` passes and replayed, so that passes shorter
    than the host's launch rate through ctypes are timed as the device runs them (every entry is enqueue-only)."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(max(1, warmup)):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(per_graph):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        reps = max(1, (steps + per_graph - 1) // per_graph)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * per_graph) * 1e-3


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def secondary_lines(shape, splits, dev):
    """Device-timed figures of the rest of the metric for the headline JSON line (N = 1): the decode kernel at 32,768 and
    131,072 tokens as a fraction of the HBM peak, the 8,192-row causal prefill and the 16/32/64-row verify passes as a
    fraction of the bf16 tensor peak.  Same timing rules as the headline: graph replays over cache copies larger than L2
    for the HBM-bound kernel; CUDA events; warm-up first."""
    from yasakani_b200 import kv4
    hbm, tf, kind = _peaks()
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    tf_sus = float(peaks.get("bf16_tflops_sustained", 1400.0))
    out = {"peak_kind": f"of {kind}"}
    side = torch.cuda.Stream(device=dev)
    q = synth.make_q(shape, 1, synth.seed_for(CONFIG_INDEX)).to(dev)

    def graph_time(fn, launches_per_graph, replays, warm):
        with torch.cuda.stream(side):
            fn(0); torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(launches_per_graph):
                    fn(i)
            for _ in range(warm):
                g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(replays):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / (replays * launches_per_graph)

    # ---- decode at the shorter contexts of the metric
    for ctx in (32768, 131072):
        max_ctx = ctx + 64
        rope = torch.empty((max_ctx, shape.rd // 2, 2), dtype=torch.float32, device=dev)
        kv4.launch_rope_table_g(rope, max_ctx, shape.theta, shape.rd)
        first = kv4.KvLayer(shape.hkv, shape.hd, max_ctx, device=dev)
        pos = torch.zeros(1, dtype=torch.int32, device=dev)
        for c in range(ctx // CHUNK):
            k, v = chunk_rows(shape, c)
            pos.fill_(c * CHUNK)
            kv4.launch_kv_append(first, k.to(dev), v.to(dev), pos, CHUNK)
        byt = shape.decode_bytes(ctx)
        n_copies = max(2, int(math.ceil(256e6 / byt)) + 1)
        layers = [first]
        for _ in range(n_copies - 1):
            l2 = kv4.KvLayer(shape.hkv, shape.hd, max_ctx, device=dev)
            for a, b in zip(l2.tensors(), first.tensors()):
                a.copy_(b)
            layers.append(l2)
        pos.fill_(ctx - 1)
        pm, pl, pacc = kv4.attn_scratch(1, splits, shape.hq, shape.hd)
        o16 = torch.empty((1, shape.hq, shape.hd), dtype=torch.float16, device=dev)
        n_graph = max(GSTEPS, n_copies)
        ext = kv4.attn_ext(early=True)
        t_attn = graph_time(lambda i: kv4.launch_attention_gqa(q, layers[i % n_copies], 1, pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, ext=ext),
                            n_graph, 8, 2)
        t_step = graph_time(lambda i: kv4.launch_decode(q, layers[i % n_copies], 1, pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, ext=ext),
                            n_graph, 8, 2)
        out[f"decode_ctx{ctx}"] = {"us_per_launch": t_attn * 1e6, "us_per_step": t_step * 1e6, "tokens_per_s": 1.0 / t_step, "bytes_per_launch": byt,
                                   "achieved_gbs": byt / t_attn / 1e9, "frac_of_hbm_peak": byt / t_attn / 1e9 / hbm, "cache_copies": n_copies}
        del layers, first, l2
        torch.cuda.empty_cache()

    # ---- multi-row passes on the tensor-core kernel
    g = torch.Generator(device=dev).manual_seed(1234)

    def tc_case(ctx, M, S):
        max_ctx = ((ctx + M + 127) // 64) * 64
        layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx, device=dev)
        pos = torch.zeros(1, dtype=torch.int32, device=dev)
        for p in range(0, ctx + M, CHUNK):
            n = min(CHUNK, ctx + M - p)
            k = torch.randn((n, shape.hkv, shape.hd), generator=g, device=dev, dtype=torch.float16)
            v = torch.randn((n, shape.hkv, shape.hd), generator=g, device=dev, dtype=torch.float16)
            pos.fill_(p)
            kv4.launch_kv_append(layer, k, v, pos, n)
        rope = torch.empty((max_ctx, shape.rd // 2, 2), dtype=torch.float32, device=dev)
        kv4.launch_rope_table_g(rope, max_ctx, shape.theta, shape.rd)
        qm = torch.randn((M, shape.hq, shape.hd), generator=g, device=dev, dtype=torch.float16)
        pos.fill_(ctx)
        pm, pl, pacc = kv4.attn_scratch(M, S, shape.hq, shape.hd)
        o16 = torch.empty((M, shape.hq, shape.hd), dtype=torch.float16, device=dev)
        ws = kv4.tc_workspace(layer, M)
        t = _timed_graph(lambda i: kv4.launch_attention_prefill_tc(qm, layer, M, pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, ws), 16, 3)
        flops = shape.attn_flops(sum(ctx + r + 1 for r in range(M)))
        res = {"us_per_pass": t * 1e6, "tflops": flops / t / 1e12, "frac_of_bf16_burst_peak": flops / t / 1e12 / tf,
               "frac_of_bf16_sustained_peak": flops / t / 1e12 / tf_sus, "splits": S, "includes": "dequant prep + attention" + ("" if S == 1 else " + merge")}
        if ctx > 0:        # a verify loop keeps the workspace: only the pass's own rows are dequantised again
            tk = _timed_graph(lambda i: kv4.launch_attention_prefill_tc(qm, layer, M, pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, ws,
                                                                        valid_tokens=ctx), 16, 3)
            res["us_per_pass_kept_workspace"] = tk * 1e6
            res["frac_of_bf16_burst_peak_kept_workspace"] = flops / tk / 1e12 / tf
        # no workspace: the attention kernel converts the packed cache itself (what the plain entries run for passes of 9..128 rows)
        tfu = _timed_graph(lambda i: kv4.launch_attention_prefill_tc(qm, layer, M, pos, S, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, None), 16, 3)
        res["us_per_pass_fused"] = tfu * 1e6
        res["frac_of_bf16_burst_peak_fused"] = flops / tfu / 1e12 / tf
        return res

    out["prefill_8192_rows"] = tc_case(0, 8192, 1)
    for M, S in ((64, 9), (32, 18), (16, 18)):
        out[f"verify_{M}_rows_ctx32768"] = tc_case(32768, M, S)
    return out


def run_secondary(args):
    from yasakani_b200 import kv4, kvx
    shape = synth.C2
    hbm, tf, kind = _peaks()
    K, W = args.steps, args.warmup
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(1234)
    base = {"n_gpus": 1, "steps": K, "warmup": W, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic"}

    def tc_case(ctx, M, splits, name, act=torch.float16):
        max_ctx = ((ctx + M + 127) // 64) * 64
        layer = kv4.KvLayer(shape.hkv, shape.hd, max_ctx)
        d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        for p in range(0, ctx + M, 8192):
            n = min(8192, ctx + M - p)
            k = torch.randn((n, shape.hkv, shape.hd), generator=g, device="cuda", dtype=torch.float16)
            v = torch.randn((n, shape.hkv, shape.hd), generator=g, device="cuda", dtype=torch.float16)
            d_pos.fill_(p)
            kv4.launch_kv_append(layer, k, v, d_pos, n)
        rope = torch.empty((max_ctx, shape.rd // 2, 2), dtype=torch.float32, device="cuda")
        kv4.launch_rope_table_g(rope, max_ctx, shape.theta, shape.rd)
        q = torch.randn((M, shape.hq, shape.hd), generator=g, device="cuda", dtype=torch.float16).to(act)
        d_pos.fill_(ctx)
        pm, pl, pacc = kv4.attn_scratch(M, splits, shape.hq, shape.hd)
        o16 = torch.empty((M, shape.hq, shape.hd), dtype=act, device="cuda")
        flops = shape.attn_flops(sum(ctx + r + 1 for r in range(M)))
        for form in ("workspace", "fused"):                        # fused: no workspace, the attention kernel converts the packed cache itself
            ws = kv4.tc_workspace(layer, M) if form == "workspace" else None
            t = _timed_graph(lambda i: kv4.launch_attention_prefill_tc(q, layer, M, d_pos, splits, pm, pl, pacc, rope, shape.hq, shape.qscale, shape.rd, o16, ws), K, W)
            nl = (2 if form == "workspace" else 1) + (0 if splits == 1 else 1)
            line = dict(base, metric="kv4_multirow_attn_tflops", value=flops / t / 1e12, unit="TFLOP/s", ms_per_step=t * 1e3, dtype="f16",
                        config={"workload": name, "form": form, "activations": "bf16" if act == torch.bfloat16 else "f16", "rows": M, "cached_tokens": ctx, "splits": splits,
                                "l2": "K/V workspace is L2-resident by design; tensor-bound" if form == "workspace" else "packed cache read once per CTA pair"},
                        gpu_launches=nl * K,
                        roofline={"bound": "tensor", "achieved": flops / t / 1e12, "peak": tf, "unit": "TFLOP/s", "frac": flops / t / 1e12 / tf, "traffic": None,
                                  "kernel": ("dequant prep + tcgen05 attention" if form == "workspace" else "tcgen05 attention with in-kernel conversion") +
                                            ("" if splits == 1 else " + merge"), "peak_kind": f"of {kind}"})
            print(json.dumps(line), flush=True)

    if args.workload == "prefill":
        tc_case(0, 8192, 1, "C5 causal prefill: 8192 rows from an empty cache, Hq24/Hkv4/hd256")
        tc_case(0, 8192, 1, "C5 causal prefill: 8192 rows from an empty cache, Hq24/Hkv4/hd256", act=torch.bfloat16)
    elif args.workload == "verify":
        for M, S in ((64, 9), (32, 18), (16, 18)):                 # splits: one wave of CTA pairs (74) over 4 kv-heads
            tc_case(32768, M, S, f"C3 verify: {M} rows against 32768 cached tokens, Hq24/Hkv4/hd256")
        tc_case(32768, 16, 18, "C3 verify: 16 rows against 32768 cached tokens, Hq24/Hkv4/hd256", act=torch.bfloat16)
    elif args.workload == "kv8":
        kvh, nh, S = shape.hkv, shape.hq, args.splits
        for ctx in (262144, 32768):
            caches = []
            for _ in range(2):
                k8 = torch.randint(-127, 128, (kvh, ctx, 256), dtype=torch.int8, device="cuda", generator=g)
                v8 = torch.randint(-127, 128, (kvh, ctx, 256), dtype=torch.int8, device="cuda", generator=g)
                caches.append((k8, v8, torch.rand((kvh, ctx), device="cuda", generator=g) * 0.03, torch.rand((kvh, ctx), device="cuda", generator=g) * 0.03))
            q = torch.randn((1, nh, 256), device="cuda", generator=g).to(torch.bfloat16)
            d_pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
            pm = torch.empty((1, S, nh), device="cuda"); pl = torch.empty_like(pm); pacc = torch.empty((1, S, nh, 256), device="cuda")
            t = _timed(lambda i: kvx.launch_kv8_attention(q, *caches[i & 1], 1, d_pos, S, pm, pl, pacc, nh), K, W)
            byt = kvh * ctx * 520
            line = dict(base, metric="kv8_decode_attn_tokens_per_s", value=1.0 / t, unit="tokens/s", ms_per_step=t * 1e3, dtype="f16",
                        config={"workload": f"Family-B decode over INT8 rows: 1 query token, Hq{nh}/Hkv{kvh}/hd256, {ctx} cached tokens", "splits": S,
                                "l2": f"2 distinct cache copies cycled; {byt / 1e6:.1f} MB read per launch (L2 is 126 MB)"},
                        gpu_launches=K,
                        roofline={"bound": "hbm", "achieved": byt / t / 1e9, "peak": hbm, "unit": "GB/s", "frac": byt / t / 1e9 / hbm, "traffic": None,
                                  "kernel": "kv8 decode attention (split-K partials)", "bytes_per_launch": byt, "peak_kind": f"of {kind}"})
            print(json.dumps(line), flush=True)
            del caches
        # verify passes over INT8 rows on the tcgen05 kernel (converter warps inside the kernel): 16 / 32 / 64 rows against 32,768 tokens
        ctx = 32768
        for M, Sv in ((64, 9), (32, 18), (16, 18)):
            mc = ((ctx + M + 127) // 64) * 64
            k8 = torch.randint(-127, 128, (kvh, mc, 256), dtype=torch.int8, device="cuda", generator=g)
            v8 = torch.randint(-127, 128, (kvh, mc, 256), dtype=torch.int8, device="cuda", generator=g)
            ks = torch.rand((kvh, mc), device="cuda", generator=g) * 0.03; vs = torch.rand((kvh, mc), device="cuda", generator=g) * 0.03
            q = torch.randn((M, nh, 256), device="cuda", generator=g).to(torch.bfloat16)
            d_pos = torch.tensor([ctx], dtype=torch.int32, device="cuda")
            pm = torch.empty((M, Sv, nh), device="cuda"); pl = torch.empty_like(pm); pacc = torch.empty((M, Sv, nh, 256), device="cuda")
            o16 = torch.empty((M, nh, 256), dtype=torch.bfloat16, device="cuda")
            def one(i):
                kvx.launch_kv8_attention_tc(q, k8, v8, ks, vs, M, d_pos, Sv, pm, pl, pacc, nh)
                kvx.launch_kv8_combine(pm, pl, pacc, Sv, M, nh, o16)
            t = _timed_graph(one, K, W)
            flops = shape.attn_flops(sum(ctx + r + 1 for r in range(M)))
            line = dict(base, metric="kv8_multirow_attn_tflops", value=flops / t / 1e12, unit="TFLOP/s", ms_per_step=t * 1e3, dtype="f16",
                        config={"workload": f"Family-B verify over INT8 rows: {M} rows against {ctx} cached tokens, Hq{nh}/Hkv{kvh}/hd256", "rows": M, "cached_tokens": ctx,
                                "splits": Sv, "l2": "INT8 rows read once per CTA pair (68 MB)"},
                        gpu_launches=2 * K,
                        roofline={"bound": "tensor", "achieved": flops / t / 1e12, "peak": tf, "unit": "TFLOP/s", "frac": flops / t / 1e12 / tf, "traffic": None,
                                  "kernel": "tcgen05 attention with in-kernel INT8 conversion + merge", "peak_kind": f"of {kind}"})
            print(json.dumps(line), flush=True)
        # decode straight over packed trellis rows (synthetic profile; groups of 4-bit trellis records): a first path on CUDA cores
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "tests", "golden"))
        from make_kvqp_blob import make_blob
        prof = kvx.TrellisProfile(make_blob())
        ctx, S = 32768, 37
        grp = torch.tensor([1, 5, 10, 14], dtype=torch.int32, device="cuda")      # 4-bit trellis records without a guard
        rows_grp = grp.repeat_interleave(ctx); rows_pos = torch.arange(ctx, dtype=torch.int32, device="cuda").repeat(kvh)
        packs = []
        for _ in range(2):
            _, pk, sk_ = kvx.tb_encode(prof, torch.randn((kvh * ctx, 256), device="cuda", generator=g), rows_grp, rows_pos)
            _, pv, sv_ = kvx.tb_encode(prof, torch.randn((kvh * ctx, 256), device="cuda", generator=g), rows_grp, rows_pos)
            packs.append((pk.view(kvh, ctx, -1), sk_.view(kvh, ctx, 2), pv.view(kvh, ctx, -1), sv_.view(kvh, ctx, 2)))
        q = torch.randn((1, nh, 256), device="cuda", generator=g).to(torch.bfloat16)
        d_pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
        pm = torch.empty((1, S, nh), device="cuda"); pl = torch.empty_like(pm); pacc = torch.empty((1, S, nh, 256), device="cuda")
        t = _timed(lambda i: kvx.launch_tb_attention(prof, q, *packs[i & 1], grp, grp, 1, d_pos, S, pm, pl, pacc, nh), K, W)
        byt = kvh * ctx * 2 * (128 + 8)                                # 4-bit payload (128 B of the 160-B row slot) + side words, K and V
        line = dict(base, metric="tb_decode_attn_tokens_per_s", value=1.0 / t, unit="tokens/s", ms_per_step=t * 1e3, dtype="f32",
                    config={"workload": f"Family-B decode over packed trellis rows (4 bits): 1 query token, Hq{nh}/Hkv{kvh}/hd256, {ctx} cached tokens",
                            "splits": S, "l2": f"2 cache copies cycled; {byt / 1e6:.1f} MB read per launch: L2-resident, the kernel is latency-bound"},
                    gpu_launches=K,
                    roofline={"bound": "hbm", "achieved": byt / t / 1e9, "peak": hbm, "unit": "GB/s", "frac": byt / t / 1e9 / hbm, "traffic": None,
                              "kernel": "tb_attn32_kernel", "bytes_per_launch": byt, "peak_kind": f"of {kind}"})
        print(json.dumps(line), flush=True)
    elif args.workload == "kvx":
        rows = 1 << 20
        x = torch.randn((rows, 256), device="cuda", generator=g)
        q8, sc = kvx.encode(x); y = torch.empty_like(x)
        for name, fn in (("encode", lambda i: kvx.encode(x, q8, sc)), ("decode", lambda i: kvx.decode(q8, sc, out=y))):
            t = _timed(fn, K, W)
            byt = rows * 1284
            line = dict(base, metric=f"kvx_{name}_rows_per_s", value=rows / t, unit="rows/s", ms_per_step=t * 1e3, dtype="f32",
                        config={"workload": f"Family-B row codec {name}: {rows} fp32 rows of 256 (rotation + INT8)", "l2": f"{byt / 1e6:.0f} MB per launch (L2 is 126 MB)"},
                        gpu_launches=K,
                        roofline={"bound": "hbm", "achieved": byt / t / 1e9, "peak": hbm, "unit": "GB/s", "frac": byt / t / 1e9 / hbm, "traffic": None,
                                  "kernel": f"kvx_{name}_kernel", "bytes_per_launch": byt, "peak_kind": f"of {kind}"})
            print(json.dumps(line), flush=True)
        # the attention block's row epilogue: M tokens of the 27B shape (24 query heads of 512 projection values, 4 + 4 KV rows)
        M, nh, kvh, rd, max_ctx = 8192, 24, 4, 64, 2 * 8192
        mk = lambda *shape: torch.randn(shape, device="cuda", generator=g).to(torch.bfloat16)
        sets = [(mk(M, nh, 512), mk(M, kvh, 256), mk(M, kvh, 256)) for _ in range(2)]            # 2 x 218 MB in: larger than L2
        qn_w, kn_w = mk(256) * 0.2, mk(256) * 0.2
        rope = torch.empty((max_ctx, rd // 2, 2), device="cuda"); kv4.launch_rope_table_g(rope, max_ctx, 1e7, rd)
        q16 = torch.empty((M, nh, 256), dtype=torch.bfloat16, device="cuda"); gate16 = torch.empty_like(q16)
        k8 = torch.empty((kvh, max_ctx, 256), dtype=torch.int8, device="cuda"); v8 = torch.empty_like(k8)
        ks = torch.empty((kvh, max_ctx), device="cuda"); vs = torch.empty_like(ks)
        d_pos = torch.tensor([4096], dtype=torch.int32, device="cuda")
        t = _timed(lambda i: kvx.launch_attn_post(*sets[i & 1], qn_w, kn_w, 1e-6, d_pos, rope, rd, q16, gate16, k8, ks, v8, vs), K, W)
        byt = M * (nh * 512 * 2 + 2 * kvh * 256 * 2 + 2 * nh * 256 * 2 + 2 * kvh * 260 + rd * 4)
        line = dict(base, metric="kvx_attn_post_tokens_per_s", value=M / t, unit="tokens/s", ms_per_step=t * 1e3, dtype="f32",
                    config={"workload": f"Family-B attention row epilogue: {M} tokens, Hq{nh}/Hkv{kvh}/hd256, rotary 64 (norm + RoPE + rotation + INT8 append)",
                            "l2": f"2 input sets cycled; {byt / 1e6:.0f} MB per launch (L2 is 126 MB)"},
                    gpu_launches=K,
                    roofline={"bound": "hbm", "achieved": byt / t / 1e9, "peak": hbm, "unit": "GB/s", "frac": byt / t / 1e9 / hbm, "traffic": None,
                              "kernel": "kvx_attn_post_kernel", "bytes_per_launch": byt, "peak_kind": f"of {kind}"})
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=262144)
    ap.add_argument("--splits", type=int, default=37, help="split-K factor; splits*Hkv = 148 = one CTA per SM")
    ap.add_argument("--cpu-sample-ctx", type=int, default=32768)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-early", action="store_true", help="do not set the `early` flag of yskn_kv4_attn_ext on the decode launches")
    ap.add_argument("--no-secondary", action="store_true", help="skip the device-timed figures of the other contexts and kernels (`secondary`)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="N > 1: how the shards' (m, l, O) triples travel")
    ap.add_argument("--e2e-copies", default="kernel", choices=["kernel", "memcpy"],
                    help="end-to-end step: host<->device copies by the library's copy kernel (default) or by cudaMemcpyAsync nodes")
    ap.add_argument("--traffic", type=float, default=None, help="dram bytes per launch from an ncu capture, if known")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "verify", "kv8", "kvx"],
                    help="decode = the headline metric (default); the others time the remaining kernels of the path on one GPU")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world, local_rank = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload != "decode":
        if rank == 0:
            run_secondary(args)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
