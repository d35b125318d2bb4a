"""Timeline of the split and combine kernels inside a replayed decode graph.

    python -m vte_b200.trace_timeline [--workload c2] [--layers 28] [--batch N] [--variant auto] [--define NAME=VALUE ...]

Builds the decode-attention cubin with -DVTEB_TRACE=1, which makes lane 0 of every warp of three
CTAs (first, middle, last but two) stamp the SM cycle counter at fixed points of the split kernel
(and %globaltimer at entry and exit), and the first and last CTA of the combine kernel stamp
%globaltimer at entry, after the dependency wait and at the end.  One traced step is run after
warm-up and the stamps are printed in microseconds relative to the first traced CTA's entry into
the first printed launch.  A development aid: the product never builds with VTEB_TRACE.
"""
from __future__ import annotations

import argparse
import ctypes

import numpy as np

from .bridge import CudaRuntime
from .compiler import CodegenEngine
from .core.decode_executor import DecodeAttentionExecutor
from .workloads import CONFIGS, draw_context_lengths

TRACE_BYTES = 1 << 20
CONSUMER = ["gt_entry", "entry", "dep_wait", "q_loaded", "first_tile", "blocks_done", "merge_bar", "stored", "exit", "gt_exit"]
LOADER = ["gt_entry", "entry", "tile1_issued", "stages_full", "last_issue", "dep_wait", "-", "-", "exit", "gt_exit"]


class DefiningCodegen(CodegenEngine):
    """Adds fixed -D macros to every kernel build."""

    def __init__(self, defines: dict):
        super().__init__()
        self.defines = dict(defines)

    def load_kernel_safe(self, hip, template_name, arch, kernel_name, **kwargs):
        return super().load_kernel_safe(hip, template_name, arch, kernel_name, **{**kwargs, **self.defines})


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2", choices=sorted(CONFIGS))
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--batch", type=int, default=0, help="keep only the first N sequences of the workload (0 = all)")
    ap.add_argument("--first", type=int, default=10, help="first launch (layer) to print")
    ap.add_argument("--count", type=int, default=3)
    ap.add_argument("--define", action="append", default=[], help="extra NAME=VALUE macro for the kernel build")
    a = ap.parse_args(argv)
    defines = {"vteb_trace": 1}
    for d in a.define:
        k, v = d.split("=", 1)
        defines[k.lower()] = int(v)

    cfg = CONFIGS[a.workload]
    lengths = draw_context_lengths(cfg)
    if a.batch:
        from dataclasses import replace
        cfg = replace(cfg, batch=min(a.batch, cfg.batch))
        lengths = lengths[:cfg.batch]
    L = a.layers
    rt = CudaRuntime(device_index=0)
    rt.initialize()
    meta = {'attention.head_count': cfg.num_q_heads, 'attention.head_count_kv': cfg.num_kv_heads,
            'attention.key_length': cfg.head_dim}
    n_kv = min(L, 28)
    ex = DecodeAttentionExecutor(rt, DefiningCodegen(defines), meta, cfg.batch, cfg.max_seq, L, n_kv_buffers=n_kv,
                                 variant=a.variant)
    trace = rt.safe_malloc(TRACE_BYTES, "trace output")
    rt.safe_memset(trace, TRACE_BYTES, "trace output")
    ex.dispatcher._external_work_ptr = trace.value          # the work words' allocation doubles as the trace buffer
    for l in range(L):
        if l < n_kv:
            ex.fill_cache_on_device(l, 100 + l, cfg.sigma_kv)
        ex.upload_layer(l, np.random.default_rng(l).standard_normal((cfg.batch, cfg.num_q_heads, cfg.head_dim),
                                                                    dtype=np.float32).astype(np.float16))
    ex.build_decode_graph()
    ex._update_staging_buffers((lengths - 1).astype(np.int32))
    rt.stream_synchronize()
    for _ in range(5):
        ex.launch_step()
    rt.synchronize()
    rt.safe_memset(trace, TRACE_BYTES, "trace output")
    rt.synchronize()
    ex.launch_step()
    rt.synchronize()
    buf = np.zeros(TRACE_BYTES // 8, dtype=np.uint64)
    rt.safe_memcpy_device_to_host(buf, trace, "trace output")
    n_split = 64 * 3 * 10 * 32
    split = buf[32:32 + n_split].reshape(64, 3, 10, 32).astype(np.int64)
    comb = buf[32 + n_split:32 + n_split + 64 * 2 * 4].reshape(64, 2, 4).astype(np.int64)
    # %globaltimer values are ~2^61 ns: subtract the origin while they are still integers
    origin = int(split[a.first, 0, 0, 0])
    for arr, slots in ((split, (0, 9)), (comb, (0, 1, 2))):
        for k in slots:
            nz = arr[..., k] != 0
            arr[..., k][nz] -= origin
    plan = ex.dispatcher._plan
    n_warps = plan.threads // 32
    cw = n_warps - 2

    def to_us(w):
        """Stamps of one warp on the global time axis (ns -> us), cycle stamps converted with the
        warp's own entry/exit pair of both clocks."""
        gt0, c0, c1, gt1 = int(w[0]), int(w[1]), int(w[8]), int(w[9])
        f = (gt1 - gt0) / max(1, c1 - c0)
        out = [gt0 / 1e3]
        for k in range(1, 9):
            out.append((gt0 + (int(w[k]) - c0) * f) / 1e3 if w[k] else float("nan"))
        out.append(gt1 / 1e3)
        tiles = []
        for i in range(8):
            if w[12 + i]:
                tiles.append(((gt0 + (int(w[12 + i]) - c0) * f) / 1e3,
                              (gt0 + (int(w[20 + i]) - c0) * f) / 1e3 if w[20 + i] else float("nan")))
        return out, f, tiles

    print(f"{a.workload} variant={a.variant} defines={defines} compact={ex.dispatcher.compact} "
          f"splits={ex.dispatcher.max_chunks} warps={n_warps} stages={plan.nstages} tile={plan.tile}")
    base = 0.0
    for l in range(a.first, min(L, a.first + a.count)):
        print(f"--- launch {l} (times in us since CTA 0 entered launch {a.first})")
        for sel, name in enumerate(("first CTA", "middle CTA", "last-but-two CTA")):
            for w in (0, cw - 1, cw, cw + 1):
                st = split[l, sel, w]
                if st[0] == 0:
                    continue
                us, f, tiles = to_us(st)
                names = CONSUMER if w < cw else LOADER
                cells = " ".join(f"{n}={u - base:7.2f}" for n, u in zip(names[1:], us[1:]) if n != "-" and u == u)
                extra = f" wait_cycles={st[11]}" if w < cw else ""
                if w < cw:
                    extra += " tiles(ready>done): " + " ".join(f"{x - base:.2f}>{y - base:.2f}" for x, y in tiles)
                elif w == cw:
                    extra += " tile issues: " + " ".join(f"{x - base:.2f}" for x, _ in tiles)
                print(f"  {name:17s} warp {w} ({'consumer' if w < cw else 'K loader' if w == cw else 'V loader'}) "
                      f"{cells}{extra} [{1e3 / f if f else 0:.0f} MHz]")
        for sel, name in enumerate(("first", "last")):
            c = comb[l, sel]
            if c[0]:
                print(f"  combine {name:5s} CTA: entry={c[0] / 1e3 - base:7.2f} dep_wait={c[1] / 1e3 - base:7.2f} end={c[2] / 1e3 - base:7.2f}")
    ex.dispatcher_check()
    ex.cleanup()
    rt.cleanup()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
