#!/usr/bin/env python3
"""Benchmark of the split-KV decode-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5]

A "step" is one decode step of attention over every layer of the workload: per
layer one split kernel and one combine kernel, all layers in one captured CUDA
graph.  The headline workload is the 32k-context single-sequence case (batch 1,
12 query / 2 KV heads of 128, 28 layers with 28 distinct KV caches = 940 MB, so
every step streams more than the 126 MB L2 holds).  It is a one-GPU workload:
with N > 1 (one process per GPU, launched by torch.distributed.run) every rank
runs its own copy and the headline value is the aggregate ("weak" scaling).

The same run also measures the workloads that do shard, and reports them under
`config.sharded` with a parity result each:

  * `c3_sequences`, `c4_sequences`: the ragged batches, sequences dealt to the
    ranks longest-first (every rank the same count), no collective;
  * `c5_kv_range_p2p`, `c5_kv_range_nccl`: one 1,048,576-position sequence whose
    KV range is split evenly over the ranks; the per-rank (o, m, l) states travel
    as tagged peer stores from the combine kernel, or through ncclAllGather.

At N = 1 the same workloads run on the one GPU, so that v_N / (N * v_1) can be
formed from the records alone.  Timing: CUDA events on the launching stream,
five trials of at least 50 ms each (a multiple of `--steps` replays), median
reported, maximum over ranks.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
import traceback
from dataclasses import replace
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from vte_b200.workloads import CONFIGS, DecodeConfig, algorithmic_bytes, draw_context_lengths, make_layer_inputs  # noqa: E402

METRIC = "decode_attention_achieved_hbm_bandwidth"
UNIT = "TB/s"
NOMINAL_PEAK_TBS = 8.0
TRIALS = 5
MIN_TRIAL_MS = 50.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the split kernel from an ncu capture,
# keyed by the content hash of the cubin that was profiled (the stem of the codegen cache file) and by
# (workload, compact CTA shape).  A rebuilt kernel has another hash and reports traffic null until it
# is captured again.
NCU_TRAFFIC_BYTES: dict[str, dict[tuple[str, bool], int]] = {
    "67b5c349857fc7c1": {("c2", True): 33621845},      # 33.62 MB read, nothing written back (partials stay in L2): three launches of the 8-layer case
}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []
        self._thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self._thread = threading.Thread(target=self._pump, daemon=True)
        self._thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def balanced_assignment(lengths, world):
    """Longest-first onto the least loaded rank, every rank getting batch / world sequences."""
    per_rank = len(lengths) // world
    load = [0] * world
    picked = [[] for _ in range(world)]
    for b in np.argsort(-lengths.astype(np.int64), kind="stable"):
        r = min((r for r in range(world) if len(picked[r]) < per_rank), key=lambda r: load[r])
        picked[r].append(int(b))
        load[r] += int(lengths[b])
    return [np.array(sorted(p), dtype=np.int64) for p in picked]


def metadata(cfg):
    return {'attention.head_count': cfg.num_q_heads, 'attention.head_count_kv': cfg.num_kv_heads,
            'attention.key_length': cfg.head_dim}


def config_json(cfg, workload, lengths, n_layers, n_kv, splits, world, extra=None):
    d = {"workload": f"{workload}: batch {cfg.batch} x {cfg.num_q_heads} query / {cfg.num_kv_heads} KV heads of "
                     f"{cfg.head_dim}, context {int(lengths.min())}..{int(lengths.max())}, {n_layers} layers "
                     f"({n_kv} distinct fp16 KV caches), fp32 accumulate and output",
         "batch_per_gpu": cfg.batch, "layers": n_layers, "distinct_kv_buffers": n_kv, "splits": splits,
         "partition": "every GPU runs its own copy (a one-GPU workload), no collective" if world > 1 else "single GPU",
         "l2_policy": "inputs larger than L2: each step streams every layer's own KV cache"}
    if extra:
        d.update(extra)
    return d


# --------------------------------------------------------------------------- timing
def timed_trials(rt, rdzv, launch, steps, trials=TRIALS, min_trial_ms=MIN_TRIAL_MS):
    """Median / min / max milliseconds per call of `launch` (which enqueues one step on the
    runtime's stream): `trials` trials, each bracketed by a barrier and a device
    synchronisation on both sides and timed with two CUDA events; a trial replays a multiple of
    `steps` steps so that it lasts at least `min_trial_ms`; every trial's time is the maximum
    over the ranks."""
    e0, e1 = rt.event_create(), rt.event_create()

    def one(n):
        rt.synchronize()
        rdzv.barrier()
        rt.event_record(e0)
        for _ in range(n):
            launch()
        rt.event_record(e1)
        rt.synchronize()
        return rdzv.max_float(rt.event_elapsed_ms(e0, e1))

    first = one(steps)
    mult = int(max(1, math.ceil(min_trial_ms / max(first, 1e-3))))
    mult = int(rdzv.max_float(float(mult)))
    per_step = sorted(one(steps * mult) / (steps * mult) for _ in range(trials))
    rt.event_destroy(e0)
    rt.event_destroy(e1)
    return {"median_ms": statistics.median(per_step), "min_ms": per_step[0], "max_ms": per_step[-1],
            "trials": trials, "replays_per_trial": steps * mult}


def cubin_hash() -> str:
    from vte_b200.compiler import CodegenEngine
    return CodegenEngine().cache_path("decode_attention", "sm_100a").stem.replace("kernel_", "")


# --------------------------------------------------------------------------- reference / CPU arm
def cpu_step(layers, threads: int):
    """One decode step of the oracle (numpy restatement of the reference's
    tools/validate_attention.py::ref_gqa_attention) over the given layers."""
    from oracle import attention_oracle as orc
    def one(layer):
        q, k, v, off = layer
        return orc.decode_attention(q, k, v, off)
    if threads <= 1:
        return [one(l) for l in layers]
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=threads) as pool:
        return list(pool.map(one, layers))


def run_reference(args, rank, world):
    if rank != 0:
        return 0
    cfg = CONFIGS[args.workload]
    lengths = draw_context_lengths(cfg)
    n_layers = args.layers or cfg.layers
    # one layer per host thread: numpy's einsum is single-threaded, layers are independent
    sample_layers = min(n_layers, max(args.cpu_layers, os.cpu_count() or 1))
    layers = [make_layer_inputs(cfg, l) for l in range(sample_layers)]
    threads = max(1, min(os.cpu_count() or 1, sample_layers))
    bytes_step = algorithmic_bytes(cfg, lengths) * sample_layers
    for _ in range(args.warmup):
        cpu_step(layers, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(layers, threads)
    dt = (time.perf_counter() - t0) / args.steps
    value = bytes_step / dt / 1e12
    sample = (f"{sample_layers} of {n_layers} layers per step, every sequence of each layer, "
              f"{threads} threads over layers (numpy einsum is single-threaded per call)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * n_layers / sample_layers,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_json(cfg, args.workload, lengths, n_layers, n_layers, None, 1),
            "us_per_layer_token": dt * 1e6 / sample_layers / cfg.batch,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


# --------------------------------------------------------------------------- sharded workloads
def _fill_sequences(rt, ex, cfg, buf, global_ids):
    """Device-side N(0, sigma) fill of one KV buffer, one seeded stream per global sequence, so a
    sequence holds the same values whichever rank owns it."""
    stride = ex.kv_batch_stride
    for i, b in enumerate(global_ids):
        seed = (cfg.base_seed * 1000 + buf) * 4096 + int(b)
        for which, cache in ((1, ex.k_cache[buf]), (2, ex.v_cache[buf])):
            rt.fill_normal_f16(ctypes.c_void_p(cache.ptr + i * stride * 2), stride, 2 * seed + which, cfg.sigma_kv,
                               cfg.outlier_frac, cfg.outlier_scale)


def _oracle_parity_of_sequences(ex, out, q_all, lengths, picks, layer=0):
    """Worst max-abs and relative-L2 error of `out[layer]` against the CPU oracle over the local
    sequences `picks`, whose cache rows are read back from the device."""
    from oracle import attention_oracle as orc
    worst_abs = worst_rel = 0.0
    for i in picks:
        n = int(lengths[i])
        k, v = ex.download_cache_rows(layer % ex.n_kv, i, n)
        ref = orc.decode_attention(q_all[layer][i:i + 1], k[None], v[None], np.array([n - 1], dtype=np.int32))
        max_abs, rel = orc.parity_metrics(out[layer][i:i + 1], ref)
        worst_abs, worst_rel = max(worst_abs, max_abs), max(worst_rel, rel)
    return worst_abs, worst_rel


def measure_sequences(args, rt, rdzv, rank, world, workload, n_layers, n_kv, steps):
    """A ragged batch sharded by sequence: every rank keeps its own sequences' caches and runs the
    same kernels on them; nothing is exchanged.  Returns the record for `config.sharded`."""
    from vte_b200.compiler import CodegenEngine
    from vte_b200.core.decode_executor import DecodeAttentionExecutor
    cfg = CONFIGS[workload]
    lengths = draw_context_lengths(cfg)
    if cfg.batch % world:
        return {"skipped": f"batch {cfg.batch} does not divide over {world} ranks"}
    mine = balanced_assignment(lengths, world)[rank] if world > 1 else np.arange(cfg.batch)
    emulated = None
    if world == 1 and getattr(args, "emulate_world", 0) > 1:
        # one rank's share of an N-rank run, alone on this GPU (the sequences partition exchanges nothing,
        # so this is what that rank would take): for tuning without N GPUs
        emulated = (args.emulate_rank, args.emulate_world)
        mine = balanced_assignment(lengths, args.emulate_world)[args.emulate_rank]
    my_lengths = lengths[mine]
    local = replace(cfg, batch=len(mine))
    ex = DecodeAttentionExecutor(rt, CodegenEngine(), metadata(cfg), local.batch, cfg.max_seq, n_layers,
                                 n_kv_buffers=n_kv, output_f32=True, variant=args.variant,
                                 num_splits=args.splits or None, min_chunk=None if args.min_chunk < 0 else args.min_chunk,
                                 balanced=False if args.no_balanced else (True if args.force_balanced else None))
    try:
        for buf in range(n_kv):
            _fill_sequences(rt, ex, cfg, buf, mine)
        q_all = np.zeros((n_layers, local.batch, cfg.num_q_heads, cfg.head_dim), dtype=np.float16)
        for l in range(n_layers):
            for i, b in enumerate(mine):
                rng = np.random.default_rng([cfg.base_seed, l, 99, int(b)])
                q_all[l, i] = rng.standard_normal((cfg.num_q_heads, cfg.head_dim), dtype=np.float32).astype(np.float16)
            ex.upload_layer(l, q_all[l])
        offsets = (my_lengths - 1).astype(np.int32)
        rt.synchronize()
        out = ex.execute_decode_batch(offsets)
        # parity: the longest and the shortest local sequence against the oracle
        picks = sorted({int(np.argmax(my_lengths)), int(np.argmin(my_lengths))})
        max_abs, rel = _oracle_parity_of_sequences(ex, out, q_all, my_lengths, picks)
        max_abs, rel = rdzv.max_float(max_abs), rdzv.max_float(rel)
        for _ in range(3):
            ex.launch_step()
        t = timed_trials(rt, rdzv, ex.launch_step, steps)
        ex.dispatcher_check()
        bytes_all = algorithmic_bytes(cfg, lengths if emulated is None else my_lengths) * n_layers
        step_s = t["median_ms"] / 1e3
        load = rdzv.allgather(str(int(my_lengths.astype(np.int64).sum())).encode())
        loads = [int(x) for x in load]
        return {
            "workload": f"{workload}: batch {cfg.batch} x {cfg.num_q_heads} query / {cfg.num_kv_heads} KV heads of {cfg.head_dim}, "
                        f"context {int(lengths.min())}..{int(lengths.max())}, {n_layers} layers per step cycling {n_kv} distinct KV caches",
            "partition": (f"{local.batch} sequences per GPU, dealt longest-first onto the least loaded GPU; no collective"
                          if world > 1 else "single GPU" if emulated is None else
                          f"rank {emulated[0]} of {emulated[1]}'s share alone on one GPU (value = this share's bytes / time)"),
            "n_gpus": world, "scaling": "strong", "value": bytes_all / step_s / 1e12, "unit": UNIT,
            "us_per_layer_step": step_s * 1e6 / n_layers, "ms_per_step": t["median_ms"],
            "ms_per_step_min_max": [t["min_ms"], t["max_ms"]], "replays_per_trial": t["replays_per_trial"],
            "positions_per_gpu_max_over_mean": max(loads) / (sum(loads) / len(loads)),
            "splits": ex.dispatcher.max_chunks, "min_chunk": ex.dispatcher.min_chunk,
            "positions_to_ctas": "equal shares of all cached positions" if ex.dispatcher.balanced else "work queue of splits",
            "kernels": "fast, compact CTAs" if ex.dispatcher.compact else "fast, full CTAs",
            "parity": {"against": "CPU oracle, layer 0, longest and shortest sequence of every rank", "max_abs": max_abs,
                       "rel_l2": rel, "within_tolerance": bool(max_abs <= 2e-3 and rel <= 1e-2)},
        }
    finally:
        ex.cleanup()


def _kv_range_small_parity(rt, rdzv, rank, world, exchange, comm):
    """The sharded path on a 16,384-position sequence with seeded host data, against the CPU
    oracle on every rank; returns the worst (max_abs, rel_l2) over ranks, layers and two replays."""
    from oracle import attention_oracle as orc
    from vte_b200.compiler import CodegenEngine
    from vte_b200.core.kv_shard import KVRangeShardedDecode, kv_range_of_rank
    total, layers = 16384, 2
    cfg = DecodeConfig("c5_small", 5, 1, 12, 2, 128, total, total, layers)
    lo, hi = kv_range_of_rank(total, rank, world)
    sh = KVRangeShardedDecode(rt, CodegenEngine(), metadata(cfg), hi - lo, layers, comm, exchange=exchange, rendezvous=rdzv)
    try:
        refs = []
        for l in range(layers):
            q, k, v, off = make_layer_inputs(cfg, l)
            sh.ex.upload_layer(l, q, np.ascontiguousarray(k[:, lo:hi]), np.ascontiguousarray(v[:, lo:hi]))
            refs.append(orc.decode_attention(q, k, v, off)[0])
        worst_abs = worst_rel = 0.0
        for _ in range(2):                      # both board parities
            out = sh.execute_decode(hi - lo - 1)
            for l in range(layers):
                max_abs, rel = orc.parity_metrics(out[l][None], refs[l][None])
                worst_abs, worst_rel = max(worst_abs, max_abs), max(worst_rel, rel)
        return rdzv.max_float(worst_abs), rdzv.max_float(worst_rel)
    finally:
        sh.cleanup()


def measure_kv_range(args, rt, rdzv, rank, world, exchange, n_layers, steps, workload="c5"):
    """One sequence whose KV range is split evenly over the ranks: per layer split -> state
    combine -> exchange of (o, m, l) -> merge, all in one graph per rank.  On one GPU the same
    sequence runs through the ordinary split + combine."""
    from vte_b200.bridge.nccl import NcclCommunicator
    from vte_b200.compiler import CodegenEngine
    from vte_b200.core.decode_executor import DecodeAttentionExecutor
    from vte_b200.core.kv_shard import KVRangeShardedDecode, kv_range_of_rank
    cfg = CONFIGS[workload]
    total = cfg.ctx_max
    lengths = np.array([total], dtype=np.int32)
    bytes_all = algorithmic_bytes(cfg, lengths) * n_layers
    name = f"{workload}: 1 x {cfg.num_q_heads} query / {cfg.num_kv_heads} KV heads of {cfg.head_dim}, context {total}, {n_layers} layer(s) per step"
    if world == 1 and getattr(args, "emulate_world", 0) > 1:
        # one rank's share of an N-rank run without its peers: split + state combine + merge of the one
        # local state; what is left of the N-rank time is the exchange
        shard = total // args.emulate_world
        sh = KVRangeShardedDecode(rt, CodegenEngine(), metadata(cfg), shard, n_layers, None, exchange="nccl", rendezvous=rdzv)
        try:
            for l in range(n_layers):
                sh.ex.fill_cache_on_device(l, cfg.base_seed * 1000 + l, cfg.sigma_kv)
                rng = np.random.default_rng([cfg.base_seed, l, 99])
                sh.ex.upload_layer(l, rng.standard_normal((1, cfg.num_q_heads, cfg.head_dim), dtype=np.float32).astype(np.float16))
            sh.execute_decode(shard - 1)
            for _ in range(3):
                sh.launch_step()
            t = timed_trials(rt, rdzv, sh.launch_step, steps)
            step_s = t["median_ms"] / 1e3
            share = algorithmic_bytes(cfg, np.array([shard], dtype=np.int32)) * n_layers
            return {"workload": name, "partition": f"one rank's share of {args.emulate_world} ({shard} positions) alone on one GPU: "
                                                   "split + state combine + merge of the local state, no exchange",
                    "n_gpus": 1, "value": share / step_s / 1e12, "unit": UNIT, "us_per_layer_step": step_s * 1e6 / n_layers,
                    "ms_per_step": t["median_ms"], "splits": sh.ex.dispatcher.max_chunks,
                    "kernels": "fast, compact CTAs" if sh.ex.dispatcher.compact else "fast, full CTAs"}
        finally:
            sh.cleanup()
    if world == 1:
        ex = DecodeAttentionExecutor(rt, CodegenEngine(), metadata(cfg), 1, total, n_layers, output_f32=True, variant=args.variant)
        try:
            q_all = np.zeros((n_layers, 1, cfg.num_q_heads, cfg.head_dim), dtype=np.float16)
            for l in range(n_layers):
                ex.fill_cache_on_device(l, cfg.base_seed * 1000 + l, cfg.sigma_kv)
                rng = np.random.default_rng([cfg.base_seed, l, 99])
                q_all[l] = rng.standard_normal(q_all[l].shape, dtype=np.float32).astype(np.float16)
                ex.upload_layer(l, q_all[l])
            offsets = np.array([total - 1], dtype=np.int32)
            rt.synchronize()
            out = ex.execute_decode_batch(offsets)
            max_abs, rel = _oracle_parity_of_sequences(ex, out, q_all, lengths, [0])
            for _ in range(3):
                ex.launch_step()
            t = timed_trials(rt, rdzv, ex.launch_step, steps)
            ex.dispatcher_check()
            step_s = t["median_ms"] / 1e3
            return {"workload": name, "partition": "single GPU (split + combine, nothing exchanged)", "n_gpus": 1,
                    "scaling": "strong", "value": bytes_all / step_s / 1e12, "unit": UNIT,
                    "us_per_layer_step": step_s * 1e6 / n_layers, "ms_per_step": t["median_ms"],
                    "ms_per_step_min_max": [t["min_ms"], t["max_ms"]], "replays_per_trial": t["replays_per_trial"],
                    "splits": ex.dispatcher.max_chunks,
                    "parity": {"against": "CPU oracle on the full 1,048,576-position sequence, layer 0", "max_abs": max_abs,
                               "rel_l2": rel, "within_tolerance": bool(max_abs <= 2e-3 and rel <= 1e-2)}}
        finally:
            ex.cleanup()

    comm = NcclCommunicator(rt, rank, world, rdzv) if exchange == "nccl" else None
    try:
        small_abs, small_rel = _kv_range_small_parity(rt, rdzv, rank, world, exchange, comm)
        lo, hi = kv_range_of_rank(total, rank, world)
        sh = KVRangeShardedDecode(rt, CodegenEngine(), metadata(cfg), hi - lo, n_layers, comm, exchange=exchange, rendezvous=rdzv)
        try:
            for l in range(n_layers):
                sh.ex.fill_cache_on_device(l, cfg.base_seed * 1000 + l * world + rank, cfg.sigma_kv)
                rng = np.random.default_rng([cfg.base_seed, l, 99])
                sh.ex.upload_layer(l, rng.standard_normal((1, cfg.num_q_heads, cfg.head_dim), dtype=np.float32).astype(np.float16))
            out = sh.execute_decode(hi - lo - 1)
            # full size: every rank must hold the same merged output, bit for bit
            digests = rdzv.allgather(hashlib.sha256(np.ascontiguousarray(out).tobytes()).digest())
            ranks_agree = all(d == digests[0] for d in digests) and bool(np.all(np.isfinite(out)))
            for _ in range(3):
                sh.launch_step()
            t = timed_trials(rt, rdzv, sh.launch_step, steps)
            sh.ex.dispatcher_check()
            step_s = t["median_ms"] / 1e3
            how = ("ncclAllGather of the states, then a merge launch" if exchange == "nccl" else
                   "tagged 64-bit peer stores over NVLink from the state combine, which also merges" if sh.tagged else
                   "peer stores over NVLink, then flags, then a merge launch")
            return {"workload": name,
                    "partition": f"KV range split evenly over {world} GPUs ({hi - lo} positions each); {how}; "
                                 f"{sh.state_floats * 4} bytes per rank per layer",
                    "n_gpus": world, "scaling": "strong", "value": bytes_all / step_s / 1e12, "unit": UNIT,
                    "us_per_layer_step": step_s * 1e6 / n_layers, "ms_per_step": t["median_ms"],
                    "ms_per_step_min_max": [t["min_ms"], t["max_ms"]], "replays_per_trial": t["replays_per_trial"],
                    "splits_per_gpu": sh.ex.dispatcher.max_chunks,
                    "parity": {"against": "CPU oracle on a 16,384-position sequence sharded the same way (every rank, 2 layers, "
                                          "2 replays); at full size all ranks' merged outputs are compared bit for bit",
                               "max_abs": small_abs, "rel_l2": small_rel, "ranks_agree_at_full_size": ranks_agree,
                               "within_tolerance": bool(small_abs <= 2e-3 and small_rel <= 1e-2 and ranks_agree)}}
        finally:
            sh.cleanup()
    finally:
        if comm is not None:
            comm.destroy()


def guarded(rdzv, fn, *a, **k):
    """Runs one sharded measurement; a failure becomes an `error` record instead of ending the run.
    A rank that fails closes its rendezvous sockets, so the ranks blocked in a collective with it fail
    at once (instead of waiting for a timeout) and the remaining sharded measurements are skipped."""
    if getattr(rdzv, "broken", False):
        return {"skipped": "an earlier sharded measurement failed on some rank"}
    try:
        rec = fn(*a, **k)
        errs = [x.decode() for x in rdzv.allgather(b"")]
        if not any(errs):
            return rec
        err = "; ".join(f"rank {r}: {x}" for r, x in enumerate(errs) if x)
    except Exception as e:                                   # noqa: BLE001
        err = f"{type(e).__name__}: {e}"
        traceback.print_exc(file=sys.stderr)
    rdzv.broken = True
    rdzv.close()
    return {"error": err[:600]}


def sharded_block(args, rt, rdzv, rank, world):
    steps = max(5, min(args.steps, 20))
    out = {}
    out["c3_sequences"] = guarded(rdzv, measure_sequences, args, rt, rdzv, rank, world, "c3", 8, 4, steps)
    out["c4_sequences"] = guarded(rdzv, measure_sequences, args, rt, rdzv, rank, world, "c4", 4, 4, steps)
    # four layers (four distinct caches) per step, as a model's decode step holds many: a graph of one
    # layer pays a graph boundary per layer (one GPU: 167.6 against 157.1 us per layer)
    if world == 1:
        out["c5_kv_range"] = guarded(rdzv, measure_kv_range, args, rt, rdzv, rank, world, "p2p", 4, steps)
    elif world <= 8:
        out["c5_kv_range_p2p"] = guarded(rdzv, measure_kv_range, args, rt, rdzv, rank, world, "p2p", 4, steps)
        out["c5_kv_range_nccl"] = guarded(rdzv, measure_kv_range, args, rt, rdzv, rank, world, "nccl", 4, steps)
    return out


# --------------------------------------------------------------------------- GPU arm
def run_ours(args, rank, world, local_rank):
    from vte_b200.bridge import CudaRuntime
    from vte_b200.bridge.rendezvous import Rendezvous
    from vte_b200.compiler import CodegenEngine
    from vte_b200.core.decode_executor import DecodeAttentionExecutor
    from vte_b200 import build as vbuild

    if rank == 0:
        vbuild.build_library()
        vbuild.build_cubins()
    rdzv = Rendezvous.from_env(timeout_s=300.0) if world > 1 else Rendezvous(0, 1)
    rdzv.barrier()

    rt = CudaRuntime(device_index=local_rank)
    rt.initialize()
    partition = args.partition or "replicas"
    if world == 1 and not (partition in ("sequences", "kv-range") and args.emulate_world > 1):
        partition = "single GPU"
    if partition in ("sequences", "kv-range"):
        # one sharded workload as the line's own value
        n_layers = args.layers or CONFIGS[args.workload].layers
        if partition == "sequences":
            rec = guarded(rdzv, measure_sequences, args, rt, rdzv, rank, world, args.workload, n_layers,
                          args.kv_buffers or min(n_layers, 4), args.steps)
        else:
            rec = guarded(rdzv, measure_kv_range, args, rt, rdzv, rank, world, args.exchange, n_layers, args.steps, args.workload)
        if rank == 0:
            line = {"metric": METRIC, "value": rec.get("value"), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                    "warmup": 3, "ms_per_step": rec.get("ms_per_step"), "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic", "config": rec}
            print(json.dumps(line), flush=True)
        rt.cleanup()
        if not getattr(rdzv, "broken", False):
            rdzv.barrier()
            rdzv.close()
        return 0

    cfg = CONFIGS[args.workload]
    lengths = draw_context_lengths(cfg)
    n_layers = args.layers or cfg.layers
    free_b, total_b = rt.get_real_mem_info()
    kv_layer_bytes = 2 * cfg.batch * cfg.kv_batch_stride * 2
    n_kv = max(1, min(n_layers, int(free_b * 0.6) // kv_layer_bytes))
    if args.kv_buffers:
        n_kv = min(n_kv, args.kv_buffers)
    ex = DecodeAttentionExecutor(rt, CodegenEngine(), metadata(cfg), cfg.batch, cfg.max_seq, n_layers,
                                 n_kv_buffers=n_kv, num_splits=args.splits or None, output_f32=True,
                                 min_chunk=None if args.min_chunk < 0 else args.min_chunk,
                                 programmatic=not args.no_pdl, compat=args.compat,
                                 prefetch_next_layer=not args.no_prefetch,
                                 fused_combine=args.fuse, variant=args.variant, rope=args.rope,
                                 rope_theta=cfg.rope_theta or 1e6, tensor_maps=not args.no_tma,
                                 balanced=False if args.no_balanced else (True if args.force_balanced else None))
    # ---- inputs: seeded host generation when it is cheap, device-side fill otherwise
    host_layers = {}
    q_all = np.zeros((n_layers, cfg.batch, cfg.num_q_heads, cfg.head_dim), dtype=np.float16)
    host_gen = kv_layer_bytes * n_kv <= (2 << 30) and not args.device_fill
    for l in range(n_layers):
        if host_gen and l < n_kv:
            q, k, v, off = make_layer_inputs(cfg, l)
            ex.upload_layer(l, q, k, v)
            if l == 0:
                host_layers[0] = (q, k, v, off)
            q_all[l] = q
        else:
            if l < n_kv:
                ex.fill_cache_on_device(l, cfg.base_seed * 1000 + l, cfg.sigma_kv, cfg.outlier_frac, cfg.outlier_scale)
            rng = np.random.default_rng([cfg.base_seed, l, 99])
            q_all[l] = rng.standard_normal(q_all[l].shape, dtype=np.float32).astype(np.float16)
            ex.upload_layer(l, q_all[l])
    offsets = (lengths - 1).astype(np.int32)
    rt.synchronize()
    ex.build_decode_graph()
    ex._update_staging_buffers(offsets)
    rt.stream_synchronize()

    bytes_step = algorithmic_bytes(cfg, lengths) * n_layers          # this rank's copy
    bytes_all = bytes_step * world
    # ---- parity of what is being timed (layer 0 against the oracle)
    parity = None
    out = ex.execute_decode_batch(offsets)
    if args.rope != "off":
        # the step rewrites the last cache row and rotates its inputs: checked by the GPU tests instead
        parity = {"skipped": "rotation modes are checked against the oracle by the GPU tests"}
    elif 0 in host_layers:
        from oracle import attention_oracle as orc
        q, k, v, off = host_layers[0]
        max_abs, rel = orc.parity_metrics(out[0], orc.decode_attention(q, k, v, off))
        parity = {"layer": 0, "max_abs": max_abs, "rel_l2": rel, "within_tolerance": bool(max_abs <= 2e-3 and rel <= 1e-2)}

    # ---- device-resident timing: graph replays between two events, five trials, median
    warm = max(3, args.warmup)
    for _ in range(warm):
        ex.launch_step()
    rt.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    t = timed_trials(rt, rdzv, ex.launch_step, args.steps, trials=args.trials, min_trial_ms=args.min_trial_ms)
    ex.dispatcher_check()

    # ---- end to end through the public call: host Q + offsets in, outputs back, every step
    for _ in range(3):
        ex.execute_decode_batch(offsets, q_host=q_all)
    e2e_trials = []
    e2e_steps = max(args.steps, int(math.ceil(args.min_trial_ms / max(t["median_ms"], 1e-3))))
    for _ in range(args.trials):
        rdzv.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ex.execute_decode_batch(offsets, q_host=q_all)
        e2e_trials.append(rdzv.max_float(time.perf_counter() - t0) / e2e_steps)
    e2e_s = statistics.median(e2e_trials)

    # ---- per-kernel durations: the same launches with an event before and after each kind of kernel
    reps = 20 if args.min_trial_ms > 0 else 2
    kern = kernel_durations(rt, ex, n_layers, reps=reps)
    probe_us = read_probe_us(rt, ex, n_layers, reps=reps) if cfg.batch == 1 else None
    clocks = sampler.stop()

    result = None
    if rank == 0:
        peak_gbs, peak_kind = measured_peaks()
        step_s = t["median_ms"] / 1e3
        value = bytes_all / step_s / 1e12
        e2e_value = bytes_all / e2e_s / 1e12
        split_bytes = bytes_step / n_layers
        split_s = kern["split_us"] * 1e-6
        achieved = split_bytes / split_s / 1e9
        layer_us = step_s * 1e6 / n_layers
        traffic = None
        if not (args.compat or args.layers):
            traffic = NCU_TRAFFIC_BYTES.get(cubin_hash(), {}).get((args.workload, ex.dispatcher.compact))
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": step_s * 1e3, "ms_per_step_min_max": [t["min_ms"], t["max_ms"]], "trials": t["trials"],
            "replays_per_trial": t["replays_per_trial"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
            "config": config_json(cfg, args.workload, lengths, n_layers, n_kv, ex.dispatcher.max_chunks, world,
                                  {"input_generation": "host, seeded" if host_gen else "device fill (counter-based normal)",
                                   "programmatic_dependent_launch": not args.no_pdl,
                                   "kv_tile_copies": "tensor-map (TMA) boxes for whole tiles, 16-byte cp.async for ragged ends" if ex.dispatcher.tensor_maps else "16-byte cp.async",
                                   "next_layer_l2_prefetch": not args.no_prefetch and cfg.batch == 1,
                                   "combine": "inside the split launch (grid barrier)" if ex.dispatcher.fused_combine else "separate launch", "kernels": "compat" if args.compat else ("fast, compact CTAs" if ex.dispatcher.compact else "fast, full CTAs"),
                                   "step_contents": {"off": "split + combine per layer",
                                                     "separate": "rotation launch + cache append + split + combine per layer",
                                                     "fused": "cache append with K rotation + split with Q rotation + combine per layer",
                                                     "fused-append": "split (with Q rotation, K rotation and the cache append) + combine per layer"}[args.rope]}),
            "us_per_layer_token": layer_us / cfg.batch,
            "pct_of_nominal_8TBs": 100.0 * value / world / NOMINAL_PEAK_TBS,
            "pct_of_measured_copy": 100.0 * value / world / (peak_gbs / 1e3),
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": int(q_all.nbytes + offsets.nbytes),
                    "d2h_bytes_per_step": int(n_layers * ex.out_bytes),
                    "ms_per_step": e2e_s * 1e3, "ms_per_step_min_max": [min(e2e_trials) * 1e3, max(e2e_trials) * 1e3],
                    "steps_per_trial": e2e_steps, "trials": args.trials,
                    "note": "KV cache is persistent device state, as in the reference's executors; per step the host "
                            "sends every layer's Q and the kv offsets and reads every layer's output"},
            "gpu_launches": ex.kernel_launches_per_step * t["replays_per_trial"] * t["trials"],
            "gpu_launches_per_step": ex.kernel_launches_per_step,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                         "frac": achieved / peak_gbs, "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})",
                         "traffic": traffic, "cubin": cubin_hash(),
                         "kernel": kern["split_name"], "kernel_us": kern["split_us"],
                         "combine_us": kern["combine_us"], "layer_us": layer_us,
                         "combine_net_us": layer_us - kern["split_us"],
                         "read_probe_us": probe_us,
                         "read_probe": "a kernel that only reads the same bytes per launch with 128-bit loads, four CTAs per SM, "
                                       "launched the same way (one launch per layer in a graph, plain stream order)",
                         "algorithmic_bytes_per_launch": int(split_bytes)},
            "clocks": clocks, "parity": parity,
        }
    ex.cleanup()

    # ---- the workloads that shard, measured in the same run
    if args.workload == "c2" and not args.no_sharded and not args.layers and args.rope == "off" and not args.compat:
        sharded = sharded_block(args, rt, rdzv, rank, world)
        if rank == 0:
            result["config"]["sharded"] = sharded

    # ---- CPU baseline on rank 0 at N = 1 only
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample_layers = min(n_layers, args.cpu_layers)
        layers = [host_layers[0]] if (0 in host_layers and sample_layers == 1) else \
                 [make_layer_inputs(cfg, l) for l in range(sample_layers)]
        best = float("inf")
        for _ in range(3):
            t0 = time.perf_counter()
            cpu_step(layers, 1)
            best = min(best, time.perf_counter() - t0)
        result["cpu_baseline"] = {
            "value": bytes_step / n_layers * sample_layers / best / 1e12, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"{sample_layers} of {n_layers} layers, best of 3, numpy restatement of "
                      f"tools/validate_attention.py::ref_gqa_attention, host has {os.cpu_count()} cores",
            "ms_per_layer": best * 1e3 / sample_layers}
    rt.cleanup()
    if not getattr(rdzv, "broken", False):
        rdzv.barrier()
        rdzv.close()
    if rank == 0:
        print(json.dumps(result), flush=True)
    return 0


def kernel_durations(rt, ex, n_layers, reps=20):
    """Average launch duration of the split kernel and of the combine kernel.
    CUDA events cannot bracket one kernel inside a replayed graph, so each kernel
    is captured into a graph of its own (every layer's launch of that kernel, in
    layer order, plain stream serialisation) and the graph is timed with events
    on the launching stream: duration = elapsed / (replays * layers), which
    includes the in-graph launch gap between consecutive kernels."""
    disp = ex.dispatcher
    name = "flash_attention_split_kv_partial_kernel" if disp.compat else disp.split_kernel_name
    out = {}
    kinds = ((0, "split_us"),) if disp.fused_combine else ((0, "split_us"), (1, "combine_us"))
    out["combine_us"] = 0.0
    for which, key in kinds:
        rt.stream_begin_capture()
        try:
            for l in range(n_layers):
                launches = disp.build_launches(l, ex.tensor_mapping, ex.offsets.ptr, batch=ex.B)
                if not disp.fuse_append:
                    launches = launches[1:]                     # drop the append launch
                fn, args, grid, block, smem = launches[which]
                if (which == 0 and not disp.compat and not disp.fused_combine
                        and ex.B * disp._plan.n_hgroups * disp.max_chunks > grid[0]):
                    # more items than CTAs: the work-queue ticket, normally cleared by the
                    # combine launch, has to start from zero
                    rt.memset_async(ctypes.c_void_p(disp.work_ptr), 4, 0, "attn_splitkv_work")
                rt.launch_kernel_recorded(fn, args, grid, block, smem)
        finally:
            graph = rt.stream_end_capture()
        out[key] = _time_graph(rt, graph, reps) / n_layers
    out["split_name"] = name
    return out


def _time_graph(rt, graph, reps):
    """Microseconds per replay of `graph` (destroyed here): 3 warm-up replays, then `reps` timed."""
    gexec = rt.graph_instantiate(graph)
    rt.graph_destroy(graph)
    e0, e1 = rt.event_create(), rt.event_create()
    for _ in range(3):
        rt.graph_launch(gexec)
    rt.synchronize()
    rt.event_record(e0)
    for _ in range(reps):
        rt.graph_launch(gexec)
    rt.event_record(e1)
    rt.synchronize()
    us = rt.event_elapsed_ms(e0, e1) * 1e3 / reps
    rt.graph_exec_destroy(gexec)
    rt.event_destroy(e0)
    rt.event_destroy(e1)
    return us


def read_probe_us(rt, ex, n_layers, reps=20):
    """What a launch that does nothing but read one layer's K and V costs: per layer one
    launch of the read-only probe over as many bytes as that layer's caches hold (two
    neighbouring cache buffers, so every launch reads its own memory), in a graph."""
    pairs = ex.n_kv // 2
    if pairs < 1 or ex.k_cache[1].ptr != ex.k_cache[0].ptr + ex.kv_bytes:
        return None
    sink = rt.safe_malloc(4 * 4096, "probe sink output")
    rt.safe_memset(sink, 4 * 4096, "probe sink output")
    regions = [c[2 * i].ptr for c in (ex.k_cache, ex.v_cache) for i in range(pairs)
               if c[2 * i + 1].ptr == c[2 * i].ptr + ex.kv_bytes]
    if not regions:
        rt.safe_free(sink, "probe sink output")
        return None
    rt.stream_begin_capture()
    try:
        for l in range(n_layers):
            rt.read_bandwidth_probe(ctypes.c_void_p(regions[l % len(regions)]), 2 * ex.kv_bytes, sink, 4 * rt.get_num_cus())
    finally:
        graph = rt.stream_end_capture()
    us = _time_graph(rt, graph, reps) / n_layers
    rt.safe_free(sink, "probe sink output")
    return us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count")
    ap.add_argument("--kv-buffers", type=int, default=0, help="distinct KV caches to cycle through")
    ap.add_argument("--splits", type=int, default=0, help="split count (0 = dispatcher's choice)")
    ap.add_argument("--min-chunk", type=int, default=-1, help="minimum positions per split (-1 = dispatcher's choice)")
    ap.add_argument("--force-balanced", action="store_true", help="equal shares per CTA even with --splits given")
    ap.add_argument("--no-balanced", action="store_true",
                    help="several sequences: splits from a work queue instead of equal shares of all positions per CTA")
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers in the CPU baseline sample")
    ap.add_argument("--partition", default="", choices=["", "replicas", "sequences", "kv-range"],
                    help="what the line's own value measures with N > 1: replicas (each rank its own copy of the workload, weak; "
                         "default), sequences (the batch is dealt to the ranks, strong), kv-range (one sequence's KV range "
                         "split over the ranks).  The default run reports the last two under config.sharded as well.")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "p2p-flags", "nccl"], help="kv-range partition: how the states travel")
    ap.add_argument("--no-sharded", action="store_true", help="skip the config.sharded measurements")
    ap.add_argument("--trials", type=int, default=TRIALS, help="timed trials (median reported)")
    ap.add_argument("--min-trial-ms", type=float, default=MIN_TRIAL_MS,
                    help="a trial replays a multiple of --steps until it lasts this long (0: exactly --steps; for profiler runs)")
    ap.add_argument("--emulate-world", type=int, default=0, help="with --partition sequences on one GPU: run only the share "
                    "that rank --emulate-rank of this many ranks would own")
    ap.add_argument("--emulate-rank", type=int, default=0)
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--variant", default="auto", choices=["full", "compact", "auto"], help="CTA shape of the split kernel")
    ap.add_argument("--fuse", action="store_true", help="combine inside the split launch (grid barrier) instead of a separate launch")
    ap.add_argument("--no-prefetch", action="store_true", help="do not prefetch the next layer's KV into L2")
    ap.add_argument("--compat", action="store_true", help="time the reference-geometry kernels")
    ap.add_argument("--no-tma", action="store_true", help="fetch every K/V tile with 16-byte asynchronous copies (no tensor-map copies)")
    ap.add_argument("--rope", default="off", choices=["off", "separate", "fused", "fused-append"],
                    help="also run the rotary embedding and the cache append inside the step: as the standalone "
                         "rotation launch, or folded into the append (K) and the split kernel's Q load")
    ap.add_argument("--device-fill", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20          # each step is seconds of CPU work
        args.warmup = min(args.warmup, 1)
        return run_reference(args, rank, world)
    return run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    sys.exit(main())
