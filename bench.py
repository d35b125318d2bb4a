#!/usr/bin/env python3
"""Benchmark of the split-KV decode-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4]

A "step" is one decode step of attention over every layer of the workload: per
layer one split kernel and one combine kernel, all layers in one captured CUDA
graph.  The default workload is the 32k-context single-sequence case (batch 1,
12 query / 2 KV heads of 128, 28 layers with 28 distinct KV caches = 940 MB, so
every step streams more than the 126 MB L2 holds).  With N > 1 (one process per
GPU, launched by torch.distributed.run) every rank runs its own sequence(s):
sequences are independent, there is no collective on the data path, and the
reported value is the aggregate over ranks ("weak" scaling).

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from vte_b200.workloads import CONFIGS, algorithmic_bytes, draw_context_lengths, make_layer_inputs  # noqa: E402

METRIC = "decode_attention_achieved_hbm_bandwidth"
UNIT = "TB/s"
NOMINAL_PEAK_TBS = 8.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the split kernel, from the ncu
# captures summarised in profiles/split_kv_partial_compact_d128_c2_32k_ncu.md (compact CTA shape,
# the default for this workload) and profiles/split_kv_partial_d128_c2_32k_ncu.md (full shape);
# same launch size as the bench's.
NCU_TRAFFIC_BYTES = {("c2", True): 33622699, ("c2", False): 33603328}


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
         "partition": "independent sequences per GPU, no collective" if world > 1 else "single GPU",
         "l2_policy": "inputs larger than L2: each step streams every layer's own KV cache"}
    if extra:
        d.update(extra)
    return d


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
    rdzv = Rendezvous.from_env() if world > 1 else Rendezvous(0, 1)
    rdzv.barrier()

    cfg = CONFIGS[args.workload]
    lengths = draw_context_lengths(cfg)
    n_layers = args.layers or cfg.layers
    partition = args.partition or "replicas"
    if world == 1:
        partition = "single GPU"
    if partition == "kv-range":
        return run_kv_range(args, rank, world, local_rank, rdzv, cfg, n_layers)
    global_cfg, global_lengths = cfg, lengths
    if partition == "sequences":
        from dataclasses import replace
        from vte_b200.core.kv_shard import sequences_of_rank
        first, last = sequences_of_rank(cfg.batch, rank, world)
        if last <= first:
            raise SystemExit(f"rank {rank} got no sequence: batch {cfg.batch} over {world} ranks")
        if args.balance and cfg.batch % world == 0:
            mine = balanced_assignment(lengths, world)[rank]
            lengths = lengths[mine]
        else:
            lengths = lengths[first:last]
        cfg = replace(cfg, batch=len(lengths))
    rt = CudaRuntime(device_index=local_rank)
    rt.initialize()
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
                                 rope_theta=cfg.rope_theta or 1e6, tensor_maps=not args.no_tma)
    # ---- inputs: seeded host generation when it is cheap, device-side fill otherwise
    host_layers = {}
    q_all = np.zeros((n_layers, cfg.batch, cfg.num_q_heads, cfg.head_dim), dtype=np.float16)
    host_gen = kv_layer_bytes * n_kv <= (2 << 30) and not args.device_fill and partition != "sequences"
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

    bytes_step = algorithmic_bytes(cfg, lengths) * n_layers          # this rank's share
    bytes_all = (algorithmic_bytes(global_cfg, global_lengths) * n_layers if partition == "sequences"
                 else bytes_step * world)
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

    # ---- device-resident timing: K graph replays between two events
    for _ in range(max(3, args.warmup)):
        ex.launch_step()
    rt.synchronize()
    rdzv.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = rt.event_create(), rt.event_create()
    rt.synchronize()
    rt.event_record(e0)
    for _ in range(args.steps):
        ex.launch_step()
    rt.event_record(e1)
    rt.synchronize()
    ms = rt.event_elapsed_ms(e0, e1)
    rdzv.barrier()
    ex.dispatcher_check()
    ms_max = rdzv.max_float(ms)

    # ---- end to end through the public call: host Q + offsets in, outputs back, every step
    for _ in range(3):
        ex.execute_decode_batch(offsets, q_host=q_all)
    rdzv.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ex.execute_decode_batch(offsets, q_host=q_all)
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    e2e_s = rdzv.max_float(e2e_s)

    # ---- per-kernel durations: the same launches with an event before and after each split kernel
    kern = kernel_durations(rt, ex, n_layers, reps=3)

    result = None
    if rank == 0:
        peak_gbs, peak_kind = measured_peaks()
        step_s = ms_max / 1e3 / args.steps
        value = bytes_all / step_s / 1e12
        e2e_value = bytes_all / (e2e_s / args.steps) / 1e12
        split_bytes = bytes_step / n_layers
        split_s = kern["split_us"] * 1e-6
        achieved = split_bytes / split_s / 1e9
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "strong" if partition == "sequences" else "weak", "vs_baseline": None,
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
            "us_per_layer_token": step_s * 1e6 / n_layers / global_cfg.batch,
            "pct_of_nominal_8TBs": 100.0 * value / world / NOMINAL_PEAK_TBS,
            "pct_of_measured_copy": 100.0 * value / world / (peak_gbs / 1e3),
            "e2e": {"value": e2e_value, "unit": UNIT,
                    "h2d_bytes_per_step": int(q_all.nbytes + offsets.nbytes),
                    "d2h_bytes_per_step": int(n_layers * ex.out_bytes),
                    "ms_per_step": e2e_s / args.steps * 1e3,
                    "note": "KV cache is persistent device state, as in the reference's executors; per step the host "
                            "sends every layer's Q and the kv offsets and reads every layer's output"},
            "gpu_launches": ex.kernel_launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                         "frac": achieved / peak_gbs, "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})",
                         "traffic": NCU_TRAFFIC_BYTES.get((args.workload, ex.dispatcher.compact)) if not (args.compat or args.layers) else None,
                         "kernel": kern["split_name"], "kernel_us": kern["split_us"],
                         "combine_us": kern["combine_us"], "algorithmic_bytes_per_launch": int(split_bytes)},
            "clocks": clocks, "parity": parity,
        }
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
    ex.cleanup()
    rt.cleanup()
    rdzv.barrier()
    rdzv.close()
    if rank == 0:
        print(json.dumps(result), flush=True)
    return 0


def run_kv_range(args, rank, world, local_rank, rdzv, cfg, n_layers):
    """One sequence whose KV range is split evenly over the ranks: per layer split ->
    state combine -> NCCL all-gather of (o, m, l) -> merge, all in one graph per rank."""
    from vte_b200.bridge import CudaRuntime
    from vte_b200.bridge.nccl import NcclCommunicator
    from vte_b200.compiler import CodegenEngine
    from vte_b200.core.kv_shard import KVRangeShardedDecode, kv_range_of_rank
    if cfg.batch != 1:
        raise SystemExit("kv-range partition is for a single sequence")
    total = cfg.ctx_max
    lo, hi = kv_range_of_rank(total, rank, world)
    rt = CudaRuntime(device_index=local_rank)
    rt.initialize()
    comm = NcclCommunicator(rt, rank, world, rdzv) if args.exchange == "nccl" else None
    sh = KVRangeShardedDecode(rt, CodegenEngine(), metadata(cfg), hi - lo, n_layers, comm, num_splits=args.splits or None,
                              programmatic=not args.no_pdl, exchange=args.exchange, rendezvous=rdzv)
    for l in range(n_layers):
        sh.ex.fill_cache_on_device(l, cfg.base_seed * 1000 + l * world + rank, cfg.sigma_kv)
        rng = np.random.default_rng([cfg.base_seed, l, 99])
        sh.ex.upload_layer(l, rng.standard_normal((1, cfg.num_q_heads, cfg.head_dim), dtype=np.float32).astype(np.float16))
    out = sh.execute_decode(hi - lo - 1)
    finite = bool(np.all(np.isfinite(out)))
    for _ in range(max(3, args.warmup)):
        sh.launch_step()
    rt.synchronize()
    rdzv.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = rt.event_create(), rt.event_create()
    rt.event_record(e0)
    for _ in range(args.steps):
        sh.launch_step()
    rt.event_record(e1)
    rt.synchronize()
    ms = rdzv.max_float(rt.event_elapsed_ms(e0, e1))
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sh.execute_decode(hi - lo - 1)
    e2e_s = rdzv.max_float(time.perf_counter() - t0)
    clocks = sampler.stop()
    lengths = np.array([total], dtype=np.int32)
    bytes_all = algorithmic_bytes(cfg, lengths) * n_layers
    step_s = ms / 1e3 / args.steps
    if rank == 0:
        peak_gbs, peak_kind = measured_peaks()
        value = bytes_all / step_s / 1e12
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
                "config": config_json(cfg, args.workload, lengths, n_layers, n_layers, sh.ex.dispatcher.max_chunks, world,
                                      {"partition": f"KV range split over {world} GPUs, "
                                                    + ("NCCL all-gather" if args.exchange == "nccl" else "tagged 64-bit peer stores over NVLink from the state combine" if sh.tagged else "peer stores over NVLink, then flags")
                                                    + f" of {sh.state_floats * 4} bytes per rank per layer",
                                       "input_generation": "device fill (counter-based normal)"}),
                "us_per_layer_token": step_s * 1e6 / n_layers,
                "pct_of_nominal_8TBs": 100.0 * value / world / NOMINAL_PEAK_TBS,
                "pct_of_measured_copy": 100.0 * value / world / (peak_gbs / 1e3),
                "e2e": {"value": bytes_all / (e2e_s / args.steps) / 1e12, "unit": UNIT, "h2d_bytes_per_step": 4,
                        "d2h_bytes_per_step": int(n_layers * sh.rows * cfg.head_dim * 4)},
                "gpu_launches": sh.ex.kernel_launches_per_step * args.steps, "clocks": clocks,
                "parity": {"finite": finite, "note": "parity of this path is asserted by the tests"}}
        print(json.dumps(line), flush=True)
    sh.cleanup()
    if comm is not None:
        comm.destroy()
    rt.cleanup()
    rdzv.barrier()
    rdzv.close()
    return 0


def kernel_durations(rt, ex, n_layers, reps=10):
    """Average launch duration of the split kernel and of the combine kernel.
    CUDA events cannot bracket one kernel inside a replayed graph, so each kernel
    is captured into a graph of its own (every layer's launch of that kernel, in
    layer order, plain stream serialisation) and the graph is timed with events
    on the launching stream: duration = elapsed / (replays * layers), which
    includes the in-graph launch gap between consecutive kernels."""
    disp = ex.dispatcher
    name = ("flash_attention_split_kv_partial_kernel" if disp.compat else
            f"vteb_split_kv_partial_{'compact_' if disp.compact else ''}{'rope_' if (disp.fuse_rope or disp.fuse_append) else ''}d{disp.head_dim}_kernel")
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
        out[key] = rt.event_elapsed_ms(e0, e1) * 1e3 / (reps * n_layers)
        rt.graph_exec_destroy(gexec)
        rt.event_destroy(e0)
        rt.event_destroy(e1)
    out["split_name"] = name
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--layers", type=int, default=0, help="override the workload's layer count")
    ap.add_argument("--kv-buffers", type=int, default=0, help="distinct KV caches to cycle through")
    ap.add_argument("--splits", type=int, default=0, help="split count (0 = dispatcher's choice)")
    ap.add_argument("--min-chunk", type=int, default=-1, help="minimum positions per split (-1 = dispatcher's choice)")
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers in the CPU baseline sample")
    ap.add_argument("--partition", default="", choices=["", "replicas", "sequences", "kv-range"],
                    help="with N > 1: replicas (each rank its own copy, weak; default), sequences (the batch is split "
                         "over the ranks, strong), kv-range (one sequence's KV range split over the ranks, NCCL all-gather)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "p2p-flags", "nccl"], help="kv-range partition: how the states travel")
    ap.add_argument("--balance", action="store_true",
                    help="sequences partition: give each rank the same number of sequences but pick them "
                         "longest-first onto the least loaded rank instead of contiguous blocks")
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
