#!/usr/bin/env python
"""Benchmark of the AlignedKV decode hot path on B200: one layer of Llama-2-7B-shaped decode attention.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step = rewind the cache to 4095 cached tokens, append token 4096 of every sequence (which flushes a 64-token
block through the plane-writer kernels), then one decode step (aligned q.K^T, softmax, probe, aligned P.V).
At N > 1 (launched with torchrun, one rank per GPU) every rank owns an independent shard of (batch, head) units of
the same size - no collective is on the data path - so the job processes N x batch sequences per step.

Other workloads (--workload): `llama3-8b-gqa-decode` (batch 64, 32 query heads over 8 KV heads, 8192 cached tokens;
the batch is split across the ranks, no collective, strong scaling) and `long-context-decode` (batch 1, 32 heads,
131072 cached tokens; at N > 1 the SEQUENCE is split across the ranks and the per-rank (max, sum, output) records are
merged after one NCCL all-gather; order-free P.V kernel, because a 131072-step fp16 chain cannot be split).

Prints ONE JSON line (rank 0).  `--impl reference` times the reference's CPU path (its torch dense attention,
restated in oracle/pipeline.py) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Llama-2-7B-shaped decode attention, one layer (the configuration the metric is quoted on)
WORKLOADS = {
    # sharding: "replicate" = every rank runs the whole shape on its own data (weak scaling); "batch" = the batch is
    # split across ranks (strong); "sequence" = the cached sequence is split across ranks and merged (strong)
    "llama2-7b-layer-decode": dict(batch=8, heads=32, kv_heads=32, head_dim=128, cache_len=4096, sharding="replicate",
                                   v_mode="exact"),
    # a quarter of the batch: same kernels and per-(batch, head) work, planes still larger than L2; sized for profiler
    # captures that replay every launch many times
    "llama2-7b-layer-decode-b2": dict(batch=2, heads=32, kv_heads=32, head_dim=128, cache_len=4096,
                                      sharding="replicate", v_mode="exact"),
    "llama3-8b-gqa-decode": dict(batch=64, heads=32, kv_heads=8, head_dim=128, cache_len=8192, sharding="batch",
                                 v_mode="exact"),
    # a quarter of that batch, for profiler captures (planes 2 x 256 MiB, larger than L2)
    "llama3-8b-gqa-decode-b16": dict(batch=16, heads=32, kv_heads=8, head_dim=128, cache_len=8192, sharding="batch",
                                     v_mode="exact"),
    "long-context-decode": dict(batch=1, heads=32, kv_heads=32, head_dim=128, cache_len=131072, sharding="sequence",
                                v_mode="order_free"),
    # one rank's shard of that sequence on 8 ranks, by itself (what a sharded step costs without its exchange)
    "long-context-decode-shard8": dict(batch=1, heads=32, kv_heads=32, head_dim=128, cache_len=16384,
                                       sharding="replicate", v_mode="order_free"),
    # a quarter of that sequence: on 2 GPUs every rank holds what a rank of the full workload holds on 8
    "long-context-decode-32k": dict(batch=1, heads=32, kv_heads=32, head_dim=128, cache_len=32768, sharding="sequence",
                                    v_mode="order_free"),
    # the same with the four-phase step whose read decisions are those of one device holding the whole sequence
    "long-context-decode-exact": dict(batch=1, heads=32, kv_heads=32, head_dim=128, cache_len=131072,
                                      sharding="sequence_exact", v_mode="order_free"),
    # full random-init Llama-2-7B decoder, AlignedKV cache on every layer: prompt of 1024 uniform-random ids, then greedy
    # decoding; a step = one token per sequence through all 32 layers (cache_len = prompt length, it grows by one per step)
    "llama2-7b-decoder": dict(batch=16, heads=32, kv_heads=32, head_dim=128, cache_len=1024, sharding="replicate",
                              v_mode="exact", decoder=dict(hidden_size=4096, intermediate_size=11008,
                                                           num_hidden_layers=32, vocab_size=32000)),
}
WORKLOAD = dict(name="llama2-7b-layer-decode", **WORKLOADS["llama2-7b-layer-decode"])
OUTLIER_CHANNELS = (3, 34, 65, 96)
METRIC = "decode_attention_tokens_per_s"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="timed blocks of --steps steps repeat until this much device time (0: three blocks; profiling runs)")
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="default workload only: do not also measure the grouped-query and long-context workloads")
    ap.add_argument("--workload", default="llama2-7b-layer-decode", choices=sorted(WORKLOADS))
    ap.add_argument("--no-graphs", action="store_true",
                    help="decoder workload: launch the dense parts op by op instead of replaying CUDA graphs")
    ap.add_argument("--v-mode", default=None, choices=["exact", "order_free"],
                    help="P.V kernel: exact = the reference's token order (bit-identical), order_free = split sequence, "
                         "fp32 accumulation (default: per workload)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "peer_unfused", "collective"],
                    help="sequence-sharded workloads: how the shards' results meet - through peer memory at the end of the "
                         "step's last kernel (peer) or in a kernel of its own (peer_unfused), or an NCCL all-gather "
                         "followed by the merge kernel (auto: peer where it can be set up)")
    args = ap.parse_args()
    WORKLOAD.clear()
    WORKLOAD.update(name=args.workload, **WORKLOADS[args.workload])
    return args


# ---------------------------------------------------------------------------------------------- shared by both arms
RUN_TOKENS = 64     # consecutive decode tokens before the cache is rewound: one 64-token block of the residual buffer
SHARDING_TEXT = {
    "replicate": "(batch, kv-head) units, no collective; every rank runs the full shape",
    "batch": "batch rows split across ranks, no collective",
    "sequence": "cached sequence split across ranks; (max, sum, output) records exchanged and merged (log-sum-exp): see "
                "`exchange`",
    "sequence_exact": "cached sequence split across ranks at multiples of 4096 tokens; four-phase step (akv_shard_step) "
                      "with exchanges of chunk statistics, probe candidates, winner rows and partial outputs: read "
                      "decisions of one device holding the whole sequence",
}


def config_dict(name: str, world: int, v_mode: str | None = None) -> dict:
    """The workload as both arms report it (same keys, same values)."""
    W = WORKLOADS[name]
    Bt, Hq, H, D, L = (W[k_] for k_ in ("batch", "heads", "kv_heads", "head_dim", "cache_len"))
    sharding = W["sharding"] if (world > 1 or W["sharding"] == "sequence_exact") else "replicate"
    per_gpu = -(-Bt // world) if sharding == "batch" else Bt
    tokens = Bt * world if W["sharding"] == "replicate" else Bt
    plane_tokens = L if sharding in ("replicate", "batch") else -(-L // world)
    plane_mib = per_gpu * H * (-(-plane_tokens // 64) * 64) * D * 4 / 2 ** 20       # K + V: high byte + two nibble planes each
    return {"workload": name, "batch": Bt, "query_heads": Hq, "kv_heads": H, "head_dim": D, "cache_len": L,
            "per_gpu_batch": per_gpu, "global_batch": tokens, "pv_kernel": v_mode or W["v_mode"],
            "sharding": SHARDING_TEXT[sharding],
            "step": "one decode token of a run of %d consecutive tokens that starts with cache_len tokens cached (all of "
                    "them quantized): 63 tokens are appended to the residual buffer, the 64th flushes the 64-token block "
                    "through the plane writers; then the cache is rewound to the start of the run (akv_rollback, inside "
                    "the timed region).  Every step streams at least cache_len quantized tokens plus the residual "
                    "ones" % RUN_TOKENS,
            "l2": "inputs larger than L2 (planes about %.0f MiB per GPU)" % plane_mib}


# ---------------------------------------------------------------------------------------------- CPU baseline
def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_dense_baseline(seed: int, budget_s: float = 12.0, name: str | None = None):
    """The reference's torch dense-attention path on the host cores, on a bounded sample of the workload:
    one batch row (all heads, full cache length), repeated while the time budget lasts.  All host cores are used
    (a launcher such as torchrun sets OMP_NUM_THREADS=1 for its children; that is undone here)."""
    import torch
    from oracle.pipeline import dense_attention_torch_cpu
    W = WORKLOADS[name or WORKLOAD["name"]]
    H, D, L = W["heads"], W["head_dim"], W["cache_len"]
    torch.set_num_threads(host_cores())
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(1, L, H, D, generator=g)
    k[..., list(OUTLIER_CHANNELS)] *= 20
    k = k.half()
    v = torch.randn(1, L, H, D, generator=g).half()
    q = torch.randn(1, 1, H, D, generator=g).half()
    cores = torch.get_num_threads()
    dense_attention_torch_cpu(q, k, v)  # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 5 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        dense_attention_torch_cpu(q, k, v)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": 1.0 / med, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"1 of {W['batch']} batch rows ({H} heads x {L} cached tokens), median of {len(times)} "
                      f"runs of the reference's fp16 torch dense attention on CPU (its prefill / dense path, "
                      f"model/KVCache_AlignedKV.py:77-79,97,87-88); per-step time extrapolated from that row"}, med


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, med = cpu_dense_baseline(args.seed, budget_s=20.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": med * 1e3 * WORKLOAD["batch"],
        "higher_is_better": True, "scaling": "weak" if WORKLOAD["sharding"] == "replicate" else "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": config_dict(WORKLOAD["name"], args.gpus, args.v_mode),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs.  The sampler
    is a separate process writing to a file, so that no Python thread competes with the launching thread."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        import tempfile
        try:
            fd, self.path = tempfile.mkstemp(prefix="akv_clocks_", suffix=".csv")
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=fd,
                                         stderr=subprocess.DEVNULL)
            os.close(fd)
        except OSError:
            self.proc = None

    def stop(self, wall0: float, wall1: float):
        """Summary of the samples taken between the two wall-clock times (time.time())."""
        if self.proc is None:
            return None
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        rows_all, rows_in = [], []
        try:
            with open(self.path) as f:
                for ln in f:
                    r = [x.strip() for x in ln.split(",")]
                    if len(r) < 9:
                        continue
                    rows_all.append(r)
                    try:
                        ts = datetime.datetime.strptime(r[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    except ValueError:
                        continue
                    if wall0 - 0.5 <= ts <= wall1 + 0.5:    # the warm-up steps right before run the same load
                        rows_in.append(r)
            os.unlink(self.path)
        except OSError:
            return None
        rows = rows_in or rows_all[-3:]
        sm, reasons, mx, pw = [], set(), None, []
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
                pw.append(float(r[3]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm),
                "power_w": statistics.median(pw) if pw else None}


# ---------------------------------------------------------------------------------------------- our arm
def load_traffic_table():
    """DRAM bytes per (batch, KV head) unit and launch of the two streaming kernels, from the ncu captures summarised
    under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum of a captured launch / its units)."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            return json.load(f)["per_unit_bytes"]
    except (OSError, KeyError, ValueError):
        return {}


def reference_kernels():
    """The reference's own CUDA kernels compiled unmodified for sm_100a (oracle/_ref), or None.  Used outside the timed
    region only: as the checker of the step's output and as the `kernel to beat` timed beside ours."""
    so = os.path.join(ROOT, "oracle", "_ref", "kv_cache_cuda.so")
    if not os.path.exists(so):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("kv_cache_cuda", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class ShardedStepFailed(SystemExit):
    """A check that every rank evaluates alike (its inputs are all-reduced) failed on a sequence-sharded workload."""


def measure(name, args, ctx, min_seconds):
    """One workload on this job's ranks: returns the dict of everything measured (rank 0; None on the others)."""
    import torch
    import torch.distributed as dist
    from alignedkv_b200.decode import DecodeLayer
    from alignedkv_b200.sharded import (DecisionExactShardedDecoder, SequenceShardedDecoder, chunk_bounds, shard_batch,
                                        shard_bounds)
    rank, world, dev = ctx["rank"], ctx["world"], ctx["dev"]
    W = WORKLOADS[name]
    Bt, Hq, H, D, L = (W[k_] for k_ in ("batch", "heads", "kv_heads", "head_dim", "cache_len"))
    G = Hq // H
    sharding = W["sharding"] if world > 1 else "replicate"
    v_mode = args.v_mode or W["v_mode"]
    if sharding == "batch":
        lo, hi = shard_batch(Bt, world, rank)
        B = hi - lo
        if B == 0:
            raise SystemExit(f"batch {Bt} cannot be split over {world} ranks")
    else:
        B = Bt
    g = torch.Generator(device=dev).manual_seed(args.seed + 1000 * rank)

    def draw(tokens):
        k_ = torch.randn(B, tokens, H, D, device=dev, generator=g)
        k_[..., list(OUTLIER_CHANNELS)] *= 20
        return k_.half(), torch.randn(B, tokens, H, D, device=dev, generator=g).half()

    if sharding == "sequence":
        # rank r holds tokens [lo, hi) of the L-1 cached tokens; the last rank also takes the decode token
        seq = SequenceShardedDecoder(B, L - 1, RUN_TOKENS + 1, H, D, dev, n_q_heads=Hq, v_mode=v_mode,
                                     exchange=args.exchange)
        lo, hi = shard_bounds(L - 1, world)[rank]
        k, v = draw(hi - lo + 1)
        seq.prefill(k[:, :hi - lo].contiguous(), v[:, :hi - lo].contiguous())
        layer = seq.backend.layer
        k_tok, v_tok = k[:, hi - lo:].contiguous(), v[:, hi - lo:].contiguous()
    elif sharding == "sequence_exact" or W["sharding"] == "sequence_exact":
        # rank r holds tokens [lo, hi) of the L-1 cached tokens, lo a multiple of 4096; every rank sees the decode token
        # (it feeds the exponent maxima), the last rank stores it
        seq = DecisionExactShardedDecoder(B, L - 1, RUN_TOKENS + 1, H, D, dev, n_q_heads=Hq)
        lo, hi = chunk_bounds(L - 1, world)[rank]
        k, v = draw(hi - lo + 1)
        seq.prefill(k[:, :hi - lo].contiguous(), v[:, :hi - lo].contiguous())
        layer = seq.layer
        k_tok, v_tok = k[:, hi - lo:].contiguous(), v[:, hi - lo:].contiguous()
        if world > 1:
            dist.broadcast(k_tok, src=world - 1)
            dist.broadcast(v_tok, src=world - 1)
    else:
        seq = None
        layer = DecodeLayer(B, L + RUN_TOKENS, H, D, dev, n_q_heads=Hq, v_mode=v_mode)   # room for one run
        k, v = draw(L)
        layer.prefill(k[:, :L - 1].contiguous(), v[:, :L - 1].contiguous())
        k_tok, v_tok = k[:, L - 1:].contiguous(), v[:, L - 1:].contiguous()
    q = torch.randn(B, 1, Hq, D, device=dev, generator=torch.Generator(device=dev).manual_seed(args.seed + 7)).half()
    owner = seq if isinstance(seq, DecisionExactShardedDecoder) else layer
    snap_flush = owner.snapshot()                          # cache_len-1 tokens cached, 63 of them in the residual buffer

    def decode(q_, k_, v_):
        return seq.decode(q_, k_, v_) if seq is not None else layer.decode(q_, k_, v_)

    def step_resident():
        return decode(q, k_tok, v_tok)

    def step_flush():
        """Rewind to cache_len-1 tokens, append token cache_len (which flushes the 64-token block), decode."""
        owner.restore(snap_flush)
        return decode(q, k_tok, v_tok)

    # end-to-end number: the step's inputs (q | k | v of the new token) lie in ONE pinned host buffer and cross in
    # one copy; the result comes back to a pinned host buffer
    nq, nk = q.numel(), k_tok.numel()
    hin = torch.cat([q.flatten(), k_tok.flatten(), v_tok.flatten()]).cpu().pin_memory()
    din = torch.empty_like(hin, device=dev)
    dq, dk, dv = din[:nq].view_as(q), din[nq:nq + nk].view_as(k_tok), din[nq + nk:].view_as(v_tok)
    hout = torch.empty((B, 1, Hq, D), dtype=torch.half).pin_memory()

    def step_e2e():
        din.copy_(hin, non_blocking=True)
        out = decode(dq, dk, dv)
        hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()          # the caller reads the result on the host
        return hout

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    run = {"pos": 0, "snap": None}

    def in_run(fn):
        """One step of a run of consecutive decode tokens: after RUN_TOKENS tokens the cache is rewound to the start of
        the run (cache_len tokens cached, residual buffer empty) - inside whatever is being timed."""
        if run["pos"] == RUN_TOKENS:
            owner.restore(run["snap"])
            run["pos"] = 0
        run["pos"] += 1
        return fn()

    def timed_blocks(fn, steps, warmup, seconds, stepper):
        """Blocks of exactly `steps` steps, each bracketed by a barrier + synchronize on both sides and timed with
        CUDA events; repeated until `seconds` of device time have been measured (at least 3 blocks).  Returns, per
        block, the MAX over the ranks of the block's time, every rank's own times (on rank 0), and the library's
        launch count per block."""
        barrier()          # (ranks whose steps wait for each other start their warm-up together)
        for _ in range(warmup):
            stepper(fn)
        own, worst, counts = [], [], []
        host_us = timed_blocks.host_us = []
        t0 = time.time()
        while len(worst) < 3 or (sum(worst) < seconds * 1e3 and len(worst) < 400):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n0 = layer.launches
            h0 = time.perf_counter()
            e0.record()
            for _ in range(steps):
                stepper(fn)
            e1.record()
            host_us.append((time.perf_counter() - h0) / steps * 1e6)   # the host's share: enqueueing the block
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            counts.append(layer.launches - n0)
            barrier()
            own.append(ms)
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)       # (the same number of blocks runs on every rank)
                ms = float(t.item())
            worst.append(ms)
        t1 = time.time()
        per_rank = None
        if world > 1:
            mine = torch.tensor([min(own), statistics.median(own), max(own), statistics.median(host_us) * steps * 1e-3],
                                device=dev, dtype=torch.float64)
            allr = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(allr, mine)
            per_rank = [[round(float(x) / steps * 1e3, 2) for x in r.tolist()[:3]] for r in allr]   # us per step
            timed_blocks.host_us_per_rank = [round(float(r[3]) / steps * 1e3, 2) for r in allr]
        return worst, per_rank, t0, t1, counts

    warm = max(args.warmup, 3)
    layer.launches = 0
    # ---- the first step of a run by itself, every step (rewind + append with the flush + decode): the run's worst step
    flush_blocks, _, _, _, _ = timed_blocks(step_flush, args.steps, warm, min_seconds / 5, lambda fn: fn())
    ms_flush = statistics.median(flush_blocks)
    # such steps again with CUDA events recorded around the two streaming kernels (the events cost ~10 us per step)
    layer.reset_counters()
    for _ in range(min(2 * args.steps, 200)):
        step_flush()
    kern_in_step = layer.kernel_times()                    # median per-kernel CUDA-event brackets of that pass
    out_last = step_flush()
    torch.cuda.synchronize()
    kern = kernel_loop_times(layer, q, v_mode) or kern_in_step
    # algorithmic bytes under this step's read decisions, summed over the ranks
    acct = layer.bytes_accounting(q)
    keys = ("k_compute", "v_compute", "read", "dense")
    tot = torch.tensor([acct[k_] for k_ in keys], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tot)
    total = dict(zip(keys, (float(x) for x in tot.tolist())))
    n_tok = layer.rest_start
    # outside any timed region: is the output right, and what do the reference's kernels need on the same state
    check = validate(layer, q, k, v, out_last, G, v_mode, sharded_sequence=seq is not None and world > 1,
                     want_ref_timing=(rank == 0))

    # ---- the headline: runs of consecutive decode tokens from cache_len cached tokens (the state the step above left)
    run["snap"] = owner.snapshot()
    sampler = ClockSampler(ctx["local"])                   # every rank watches its own GPU
    sampler.start()
    blocks, per_rank, t0, t1, counts = timed_blocks(step_resident, args.steps, warm, min_seconds, in_run)   # no instrumentation inside
    host_enqueue_us = statistics.median(timed_blocks.host_us)
    host_enqueue_per_rank = getattr(timed_blocks, "host_us_per_rank", None) if world > 1 else None
    clocks = sampler.stop(t0, time.time())
    if world > 1:
        # the block time is the maximum over the ranks: the clocks and power of every rank's GPU beside its own times
        every = [None] * world
        dist.all_gather_object(every, clocks)
        if clocks is not None:
            clocks = dict(clocks, per_rank=[None if c is None else {k_: c[k_] for k_ in ("sm_mhz", "power_w", "reasons")}
                                            for c in every])
    launches = int(statistics.median(counts))              # kernels of this library per timed block (its own counter)
    # whole runs per block: all blocks are alike, take the median; else the blocks differ (some hold the flush and the
    # rewind, some do not) and the mean is the cost per token
    whole_runs = args.steps % RUN_TOKENS == 0
    ms = statistics.median(blocks) if whole_runs else sum(blocks) / len(blocks)
    e2e_blocks, _, _, _, _ = timed_blocks(step_e2e, args.steps, warm, min_seconds / 2, in_run)
    ms_e2e = statistics.median(e2e_blocks) if whole_runs else sum(e2e_blocks) / len(e2e_blocks)

    flag = torch.tensor([int(layer.lib.akv_device_error_flag())], device=dev)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    check["device_error_flag"] = int(flag.item())
    if check["device_error_flag"] != 0:
        raise (ShardedStepFailed if seq is not None and world > 1 else SystemExit)(
            "bench: a bounded wait inside a kernel gave up during the run (akv_device_error_flag != 0)")
    if seq is not None and world > 1:
        # sequence shards: no rank can check the output against the whole sequence, but every rank must hold the SAME
        # merged output, finite and not zero (a wait that ran out, or a record that did not arrive, shows here)
        mine = out_last.float().flatten().contiguous()
        first = mine.clone()
        dist.broadcast(first, src=0)
        same = torch.tensor([int(torch.equal(mine, first) and bool(torch.isfinite(mine).all()) and
                                 float(mine.abs().max()) > 0.0)], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        check["sharded_outputs_identical"] = bool(same.item())
        if not check["sharded_outputs_identical"]:
            raise ShardedStepFailed("bench: the ranks of a sequence-sharded step do not hold the same finite non-zero "
                                    "output")
    for key_, bound in (("exact_vs_ref_kernel", 1e-3), ("step_output_vs_fp32_dense", 0.1)):
        if check["accuracy"].get(key_) is not None and check["accuracy"][key_] > bound:
            raise SystemExit(f"bench: {key_} = {check['accuracy'][key_]:.3e} exceeds {bound}")
    if rank != 0:
        return None
    ms_step = ms / args.steps
    tokens = Bt * world if W["sharding"] == "replicate" else Bt
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    traffic = load_traffic_table()
    units = B * H

    def roofline_of(kname):
        if kname not in kern:
            return None
        a = acct[kname] / (kern[kname]["us"] * 1e-6) / 1e9
        tkey = "%s|group%d|%s" % (kname if not (kname == "v_compute" and v_mode == "order_free") else
                                  "v_compute_order_free", G, n_tok)
        per_unit = traffic.get(tkey)
        return {"bound": "hbm", "kernel": kname, "achieved": a, "peak": peak, "unit": "GB/s", "frac": a / peak,
                "peak_source": "of measured" if peaks else "of fallback",
                "traffic": per_unit * units if per_unit is not None else None,
                "us_per_launch": kern[kname]["us"], "algorithmic_bytes": acct[kname]}

    dom = max(kern, key=lambda n: kern[n]["us"]) if kern else None
    roofline = roofline_of(dom) if dom else None
    if roofline:
        roofline["timing"] = ("average duration of %d back-to-back launches of the kernel on the state of the timed step "
                              "(same planes, alignment inputs, probabilities, thresholds), between two CUDA events on "
                              "the launching stream, after 3 warm-up launches; the planes one launch streams are larger "
                              "than L2.  A bracket of events around a single launch inside the step adds the launch "
                              "latency after the first event (kernels_us_in_step_event_brackets)" % KERNEL_LOOP_LAUNCHES)
        roofline["other_kernel"] = roofline_of("k_compute" if dom == "v_compute" else "v_compute")
    cfg = config_dict(name, world, v_mode)
    if isinstance(seq, DecisionExactShardedDecoder):
        cfg["sharding"] = SHARDING_TEXT["sequence_exact"]
    if isinstance(seq, SequenceShardedDecoder):
        cfg["exchange"] = seq.exchange + (f" ({seq.exchange_note})" if seq.exchange_note else "")
    return {
        "metric": METRIC, "value": tokens / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak" if W["sharding"] == "replicate" else "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": cfg,
        "timing": {"blocks": len(blocks), "steps_per_block": args.steps, "block_ms_median": statistics.median(blocks),
                   "block_ms_mean": sum(blocks) / len(blocks), "statistic": "median" if whole_runs else "mean",
                   "block_ms_min": min(blocks),
                   "block_ms_max": max(blocks), "seconds_timed": sum(blocks) * 1e-3,
                   "per_rank_us_per_step_min_median_max": per_rank,
                   "host_enqueue_us_per_step": round(host_enqueue_us, 2),
                   "host_enqueue_us_per_step_per_rank": host_enqueue_per_rank,
                   "rule": "every block = exactly `steps` steps between barrier + synchronize pairs, CUDA events, max "
                           "over ranks; the reported step time is the median block when a block holds whole runs of "
                           "%d tokens (the default), else the mean over the blocks; host_enqueue_us_per_step = wall "
                           "time rank 0's host needed to enqueue a block, per step (a step whose device time is close "
                           "to it is bound by the host, not by the GPU)" % RUN_TOKENS},
        "effective_hbm_gbs": total["dense"] / (ms_step * 1e-3) / 1e9,
        "achieved_hbm_gbs": total["read"] / (ms_step * 1e-3) / 1e9,
        "bytes_read_over_dense": total["read"] / total["dense"],
        "kernels_us": {n: round(kv_["us"], 2) for n, kv_ in kern.items()},
        "kernels_us_in_step_event_brackets": {n: round(kv_["us"], 2) for n, kv_ in kern_in_step.items()},
        "roofline": roofline,
        "e2e": {"value": tokens / (ms_e2e / args.steps * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int((q.numel() + k_tok.numel() + v_tok.numel()) * 2),
                "d2h_bytes_per_step": int(hout.numel() * 2), "ms_per_step": ms_e2e / args.steps},
        "flush_step": {"ms_per_step": ms_flush / args.steps,
                       "what": "the flushing step timed by itself, every step: rewind to cache_len-1 tokens, append "
                               "token cache_len with the flush of the 64-token block, decode.  The per-kernel figures, "
                               "the accuracy block and the reference kernels' timings are taken on this step's state"},
        "gpu_launches": launches,
        "clocks": clocks,
        "accuracy": check["accuracy"],
        "validation": {"device_error_flag": check["device_error_flag"], "note": check["note"],
                       "sharded_outputs_identical": check.get("sharded_outputs_identical")},
        "ref_cuda_kernels_us": check["ref_cuda_kernels_us"],
    }


KERNEL_LOOP_LAUNCHES = 20


def kernel_loop_times(layer, q, v_mode):
    """Average launch duration of the two streaming kernels: KERNEL_LOOP_LAUNCHES back-to-back launches of each, through
    the operator entry points of the C ABI, on the state the last step left behind (the step's own planes, alignment
    inputs, probabilities and threshold bytes), between two CUDA events.  None when the state has residual tokens."""
    import math
    import torch
    from alignedkv_b200 import _lib
    B, H, Hq, G, D = layer.B, layer.H, layer.Hq, layer.G, layer.D
    qn = layer.rest_start
    if layer.rest_len != 0 or qn == 0:
        return None
    dev = q.device
    lib = layer.lib
    R = (qn // 64 + 1) * 64
    nmb = layer.k_first_8.shape[2]
    st = torch.cuda.current_stream(dev).cuda_stream
    off = {n: layer._scratch_offset(n) for n in ("kq", "kqmax", "amin")}
    p_ptr = layer.scratch.data_ptr()                       # probabilities: rows of R halves
    s_tmp = torch.empty(B * Hq * R, dtype=torch.half, device=dev)
    o_tmp = torch.empty(B * Hq * D, dtype=torch.half, device=dev)
    flags = (2 if v_mode == "order_free" else 0) | (1 if layer.reference else 0)
    nbytes = int(lib.akv_v_cache_compute_scratch_bytes(B, H, G, qn))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    base = layer.scratch.data_ptr()

    def launch_k():
        _lib.check("k_cache_compute", lib.akv_k_cache_compute_gqa(
            layer.k_first_8.data_ptr(), layer.k_mid_4.data_ptr(), layer.k_last_4.data_ptr(), base + off["kq"],
            base + off["kqmax"], q.data_ptr(), s_tmp.data_ptr(), B, H, G, qn // 64, nmb, D, 64, 1, 1.0 / math.sqrt(D),
            1 if layer.reference else 0, st))

    def launch_v():
        _lib.check("v_cache_compute", lib.akv_v_cache_compute_gqa(
            layer.v_first_8.data_ptr(), layer.v_mid_4.data_ptr(), layer.v_last_4.data_ptr(), p_ptr, base + off["amin"],
            o_tmp.data_ptr(), ws.data_ptr(), ws.numel(), B, H, G, layer.L, D, R, qn, flags, st))

    res = {}
    for name, fn in (("k_compute", launch_k), ("v_compute", launch_v)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(KERNEL_LOOP_LAUNCHES):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        res[name] = {"us": e0.elapsed_time(e1) * 1e3 / KERNEL_LOOP_LAUNCHES, "launches": KERNEL_LOOP_LAUNCHES}
    return res


def validate(layer, q, k, v, out_last, G, v_mode, sharded_sequence, want_ref_timing):
    """Outside the timed region, on the state the last step left behind: max-norm relative errors
    max|a - b| / max|b| of the step's output against fp32 dense attention over the original tensors and - where the
    reference's kernels can run (multi-head attention, their compiled extension at hand) - of the exact and the
    order-free P.V kernels against the reference kernel on the same probabilities and thresholds; and the reference
    kernels' own durations on that state (aligned, and reading every plane)."""
    import math
    import torch
    from alignedkv_b200 import _lib
    acc = {"exact_vs_ref_kernel": None, "order_free_vs_ref_kernel": None, "exact_vs_fp32_dense": None,
           "order_free_vs_fp32_dense": None, "ref_kernel_vs_fp32_dense": None, "step_output_vs_fp32_dense": None}
    res = {"accuracy": acc, "ref_cuda_kernels_us": None, "note": ""}
    if sharded_sequence:
        res["note"] = "sequence-sharded run: no rank holds the whole sequence, accuracy is covered by the tests"
        return res
    B, H, Hq, D, L = layer.B, layer.H, layer.Hq, layer.D, layer.cache_len
    dev = q.device

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max())

    # fp32 dense attention over the original fp16 tensors, one batch row at a time
    truth = torch.empty(B, 1, Hq, D, device=dev)
    for b in range(B):
        kk = k[b, :L].float().repeat_interleave(G, dim=1).transpose(0, 1)        # [Hq, L, D]
        vv = v[b, :L].float().repeat_interleave(G, dim=1).transpose(0, 1)
        s = torch.matmul(q[b, 0].float().unsqueeze(1), kk.transpose(1, 2)) / math.sqrt(D)   # [Hq, 1, L]
        truth[b, 0] = torch.matmul(torch.softmax(s, dim=-1), vv).squeeze(1)
        del kk, vv
    acc["step_output_vs_fp32_dense"] = rel(out_last, truth)
    acc["exact_vs_fp32_dense" if v_mode == "exact" else "order_free_vs_fp32_dense"] = acc["step_output_vs_fp32_dense"]
    qn = layer.rest_start
    if layer.rest_len != 0 or qn == 0:
        res["note"] = "residual tokens present: per-kernel comparison skipped"
        return res
    R = (qn // 64 + 1) * 64
    p = layer.scratch[:B * Hq * R * 2].view(B, Hq, 1, R * 2)                       # probabilities as the operators take them
    off = layer._scratch_offset("amin")
    amin = layer.scratch[off:off + B * Hq].clone()
    st = torch.cuda.current_stream(dev).cuda_stream
    lib = layer.lib
    other = torch.empty(B, 1, Hq, D, dtype=torch.half, device=dev)
    nbytes = lib.akv_v_cache_compute_scratch_bytes(B, H, G, qn)
    ws = torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=dev)
    flags = 0 if v_mode == "order_free" else 2                                     # the P.V kernel the step did NOT use
    rc = lib.akv_v_cache_compute_gqa(layer.v_first_8.data_ptr(), layer.v_mid_4.data_ptr(), layer.v_last_4.data_ptr(),
                                     p.data_ptr(), amin.data_ptr(), other.data_ptr(), ws.data_ptr(), ws.numel(), B, H, G,
                                     layer.L, D, R, qn, flags, st)
    _lib.check("v_cache_compute", rc)
    acc["order_free_vs_fp32_dense" if v_mode == "exact" else "exact_vs_fp32_dense"] = rel(other, truth)
    exact, order_free = (out_last, other) if v_mode == "exact" else (other, out_last)
    ext = reference_kernels() if G == 1 else None
    if ext is None:
        res["note"] = ("grouped-query attention: the reference's kernels assert multi-head attention" if G > 1 else
                       "the reference's compiled extension (oracle/_ref) is not at hand")
        return res
    nmb = layer.k_first_8.shape[2]
    kq_off, kqm_off = layer._scratch_offset("kq"), layer._scratch_offset("kqmax")
    kq = layer.scratch[kq_off:kq_off + B * Hq * D].view(B, 1, Hq, D)
    kqmax = layer.scratch[kqm_off:kqm_off + B * Hq].view(B, 1, Hq, 1)
    amin4 = amin.view(B, Hq, 1, 1)

    def ref_k(reference):
        return ext.k_cache_compute(layer.k_first_8, layer.k_mid_4, layer.k_last_4, kq, kqmax, q.view(torch.uint8), B, H,
                                   qn // 64, nmb, D, 64, 1, 1.0 / math.sqrt(D), reference)

    def ref_v(reference):
        return ext.v_cache_compute(layer.v_first_8, layer.v_mid_4, layer.v_last_4, p, amin4, B, H, layer.L, D, R, qn,
                                   reference)

    o_ref = ref_v(False).view(torch.half).view(B, 1, Hq, D)
    torch.cuda.synchronize()
    acc["exact_vs_ref_kernel"] = rel(exact, o_ref)
    acc["order_free_vs_ref_kernel"] = rel(order_free, o_ref)
    acc["ref_kernel_vs_fp32_dense"] = rel(o_ref, truth)
    if want_ref_timing:
        def med_us(fn):
            ts = []
            for i in range(6):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                if i > 0:
                    ts.append(e0.elapsed_time(e1) * 1e3)
            return round(statistics.median(ts), 1)
        res["ref_cuda_kernels_us"] = {
            "what": "the reference's own kernels (extension/csrc, compiled unmodified for sm_100a) on the state of the "
                    "timed step: same planes, alignment inputs, probabilities and thresholds; median of 5 launches",
            "k_compute": {"aligned": med_us(lambda: ref_k(False)), "all_planes": med_us(lambda: ref_k(True))},
            "v_compute": {"aligned": med_us(lambda: ref_v(False)), "all_planes": med_us(lambda: ref_v(True))}}
    return res


OTHER_WORKLOADS = ("llama3-8b-gqa-decode", "long-context-decode")


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: alignedkv_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from alignedkv_b200 import _lib
    _lib.load()
    ctx = dict(rank=rank, world=world, local=local, dev=dev)
    line = measure(args.workload, args, ctx, args.min_seconds)
    others = {}
    if args.workload == "llama2-7b-layer-decode" and not args.no_other_workloads:
        # the other configurations the metric is asked for, at the same number of GPUs: the grouped-query batch (batch
        # rows split across the ranks) and the long context (sequence split across the ranks, one NCCL all-gather +
        # log-sum-exp merge per step)
        for name in OTHER_WORKLOADS:
            torch.cuda.empty_cache()
            try:
                r = measure(name, args, ctx, args.min_seconds / 2)
            except ShardedStepFailed as e:
                # (every rank gets here together.)  The exchange through peer memory did not hold on this machine:
                # measure the workload with the NCCL all-gather instead and say so
                if args.exchange == "collective":
                    raise
                _lib.load().akv_device_error_clear()
                again = argparse.Namespace(**dict(vars(args), exchange="collective"))
                r = measure(name, again, ctx, args.min_seconds / 2)
                if r is not None:
                    r["config"]["exchange"] += f"; the peer-memory exchange failed first ({e})"
            if r is not None:
                others[name] = {k_: r[k_] for k_ in ("value", "unit", "ms_per_step", "scaling", "config", "kernels_us",
                                                     "roofline", "e2e", "bytes_read_over_dense", "accuracy", "timing",
                                                     "gpu_launches", "ref_cuda_kernels_us", "flush_step", "validation")}
    if rank == 0:
        if others:
            line["other_workloads"] = others
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_dense_baseline(args.seed)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_decoder(args):
    """The full-decoder workload: tokens/s of greedy decoding with the AlignedKV cache on every layer."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: alignedkv_b200 has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from alignedkv_b200.llama import LlamaConfig, LlamaDecoder

    B, Hq, H, D, S = (WORKLOAD[k_] for k_ in ("batch", "heads", "kv_heads", "head_dim", "cache_len"))
    dc = WORKLOAD["decoder"]
    cfg = LlamaConfig(hidden_size=dc["hidden_size"], intermediate_size=dc["intermediate_size"],
                      num_hidden_layers=dc["num_hidden_layers"], num_attention_heads=Hq, num_key_value_heads=H,
                      vocab_size=dc["vocab_size"])
    warm = max(args.warmup, 3)
    v_mode = args.v_mode or WORKLOAD["v_mode"]
    max_len = -(-(S + 2 * (warm + args.steps) + 2) // 64) * 64
    model = LlamaDecoder(cfg, B, max_len, dev, seed=args.seed + rank, v_mode=v_mode)
    ids = torch.randint(0, cfg.vocab_size, (B, S), device=dev,
                        generator=torch.Generator(device=dev).manual_seed(args.seed + 100 + rank))
    tok = model.prefill(ids).argmax(-1)
    if not args.no_graphs:
        model.capture_graphs()                           # the dense parts between two attention calls: one graph each
    lib = model.caches[0].lib

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    state = {"tok": tok}
    htok = torch.empty(B, dtype=torch.int64).pin_memory()
    hin = tok.cpu().pin_memory()

    def step_resident():
        state["tok"] = model.step(state["tok"]).argmax(-1)

    def step_e2e():
        t = hin.to(dev, non_blocking=True)               # the caller hands the previous tokens over from the host
        nxt = model.step(t).argmax(-1)
        htok.copy_(nxt, non_blocking=True)
        torch.cuda.current_stream().synchronize()        # and reads the new ones there
        hin.copy_(htok)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        ms = e0.elapsed_time(e1)
        barrier()
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, t0, t1

    sampler = ClockSampler(local) if rank == 0 else None
    model.caches[0].launches = 0                         # (the counter is the library's, shared by all layers)
    lib.akv_set_tuning(b"timing", 1)
    lib.akv_timing_reset()
    if sampler:
        sampler.start()
    ms, t0, t1 = timed(step_resident, args.steps, warm)
    clocks = sampler.stop(t0, t1) if sampler else None
    kern = model.caches[0].kernel_times()                 # medians over every layer's launches in the timed steps
    launches = model.caches[0].launches // (args.steps + warm)
    acct = {"k_compute": 0.0, "v_compute": 0.0, "read": 0.0, "dense": 0.0}
    for c in model.caches:                                # the last step's read decisions, every layer
        a = c.bytes_accounting()
        for k_ in acct:
            acct[k_] += a[k_]
    ms_e2e, _, _ = timed(step_e2e, args.steps, warm)
    if rank == 0:
        ms_step = ms / args.steps
        tokens = B * world
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        L_now = model.caches[0].cache_len
        nl = cfg.num_hidden_layers
        weight_bytes = 2.0 * sum(t.numel() for lyr in model.layers for t in lyr.values()) + 2.0 * model.lm_head.numel()
        dom = max(kern, key=lambda n: kern[n]["us"]) if kern else None
        roofline = None
        if dom:
            a = acct[dom] / nl / (kern[dom]["us"] * 1e-6) / 1e9     # per launch = per layer
            roofline = {"bound": "hbm", "kernel": dom, "achieved": a, "peak": peak, "unit": "GB/s", "frac": a / peak,
                        "peak_source": "measured" if peaks else "fallback", "traffic": None,
                        "us_per_launch": kern[dom]["us"], "algorithmic_bytes": acct[dom] / nl,
                        "timing": "median of CUDA-event brackets over every layer's launch in the timed steps"}
        line = {
            "metric": METRIC, "value": tokens / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic (random-init weights ~N(0,0.02), uniform-random prompt ids)",
            "config": {"workload": WORKLOAD["name"], "batch": B, "query_heads": Hq, "kv_heads": H, "head_dim": D,
                       "layers": nl, "hidden": cfg.hidden_size, "ffn": cfg.intermediate_size, "vocab": cfg.vocab_size,
                       "prompt_len": S, "cache_len_at_end": L_now, "global_batch": tokens, "pv_kernel": v_mode,
                       "step": "one greedy token per sequence through all layers (projections and MLP: fp16 cuBLAS "
                               "through torch; attention: the AlignedKV decode step of every layer)",
                       "dense_parts": "launched op by op" if args.no_graphs else
                                      "replayed from CUDA graphs, one per stretch between two attention calls",
                       "l2": "weights 13.5 GB + planes, far larger than L2"},
            "attention_kernels_us_per_layer": {n: round(kv_["us"], 2) for n, kv_ in kern.items()},
            "attention_bytes_read_over_dense": acct["read"] / acct["dense"],
            "weight_bytes_per_step": weight_bytes,
            "roofline": roofline,
            "e2e": {"value": tokens / (ms_e2e / args.steps * 1e-3), "unit": UNIT, "h2d_bytes_per_step": B * 8,
                    "d2h_bytes_per_step": B * 8, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches * args.steps,
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference_arm(args)
    elif "decoder" in WORKLOAD:
        run_decoder(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
