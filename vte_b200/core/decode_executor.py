"""Decode-step driver for the attention path: one captured CUDA graph per step.

The attention-only counterpart of `HIPGraphExecutor` / `BatchedHIPGraphExecutor`
(vte/core/hip_graph_executor.py:504-819, vte/core/batched_hip_graph_executor.py:
231-292): it owns the per-layer buffers an executor would hand the dispatcher
(`blk.{l}.q_proj.output`, `blk.{l}.k_proj.output`, `blk.{l}.v_proj.output`,
`blk.{l}.attention.output`, `blk.{l}.kv_cache.k/.v`,
`kv_batch_stride_elements`), records every layer's launches from
`SplitKVAttentionDispatcher.build_launches` into one graph
(hip_graph_executor.py:635-651), and replays it per token after rewriting the
device array of per-sequence kv offsets from a staging buffer
(hip_graph_executor.py:772-789; batched: batched_hip_graph_executor.py:276-285).
Unlike the reference's batched executor it admits ragged context lengths.
"""
from __future__ import annotations

import ctypes
import types
from typing import Optional

import numpy as np

from ..bridge.errors import CudaSafetyError
from ..bridge.memory import MemoryRegion, SlabAllocator
from ..config import ENV_NO_PDL, env_flag
from .split_kv_attention import SplitKVAttentionDispatcher


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class DecodeAttentionExecutor:
    def __init__(self, hip, codegen, metadata: dict, batch_size: int, context_length: int, n_layers: int, *,
                 n_kv_buffers: Optional[int] = None, num_splits: Optional[int] = None, output_f32: bool = True,
                 use_graph: bool = True, programmatic: Optional[bool] = None, compat: bool = False,
                 with_append: bool = False, fixed_chunk_size=None, min_chunk: Optional[int] = None,
                 strict_empty_splits: bool = False, allocator: Optional[SlabAllocator] = None,
                 emit_state: bool = False, per_layer_hook=None, prefetch_next_layer: bool = True,
                 fused_combine: Optional[bool] = None, variant: str = "auto", rope: str = "off",
                 rope_theta: float = 1e6, tensor_maps: bool = True, fuse_append: bool = False,
                 balanced: Optional[bool] = None):
        self.hip = hip
        # rope: "off" = Q and K arrive rotated; "separate" = the reference's standalone rotation
        # launch runs before the append (rotating the projections in place); "fused" = the append
        # rotates K and the split kernel rotates Q.  Either way the step includes the append.
        # "fused-append": as "fused", and the split kernel also does the append (no append launch).
        if rope not in ("off", "separate", "fused", "fused-append"):
            raise CudaSafetyError(f"rope must be off, separate, fused or fused-append, not {rope!r}")
        self.rope = rope
        if rope != "off":
            with_append = True
        self.metadata = dict(metadata)
        self.B = int(batch_size)
        self.S = int(context_length)
        self.L = int(n_layers)
        self.n_kv = int(n_kv_buffers or n_layers)   # distinct KV buffers; layers cycle through them
        if not (1 <= self.n_kv <= self.L):
            raise CudaSafetyError(f"n_kv_buffers {self.n_kv} outside 1..{self.L}")
        self.Hq = int(metadata.get('attention.head_count', 12))
        self.Hkv = int(metadata.get('attention.head_count_kv', 2))
        self.D = int(metadata.get('attention.key_length', 128))
        self.output_f32 = bool(output_f32)
        self.use_graph = bool(use_graph)
        self.programmatic = (not env_flag(ENV_NO_PDL)) if programmatic is None else bool(programmatic)
        self.with_append = bool(with_append)
        self.emit_state = bool(emit_state)          # outputs are [B, Hq, D + 2] fp32 shard states
        self.per_layer_hook = per_layer_hook        # called as hook(layer) after a layer's launches are recorded
        self.launch_rewriter = None                 # optional: rewriter(layer, launches) -> launches, before recording
        self.kv_batch_stride = self.S * self.Hkv * self.D
        if self.kv_batch_stride >= 2 ** 31:
            raise CudaSafetyError("one sequence's cache exceeds 2^31 elements: the kernel ABI's stride is an int")

        out_elem = 4 if self.output_f32 else 2
        self.kv_bytes = self.B * self.kv_batch_stride * 2           # one K (or V) cache of one layer
        self.q_bytes = self.B * self.Hq * self.D * 2
        self.kvnew_bytes = self.B * self.Hkv * self.D * 2
        self.out_bytes = self.B * self.Hq * self.D * out_elem
        if self.emit_state:
            self.out_bytes = self.B * self.Hq * (self.D + 2) * 4

        self._owns_allocator = allocator is None
        if allocator is None:
            need = (2 * self.n_kv * (self.kv_bytes + 256) + self.L * (self.q_bytes + 2 * self.kvnew_bytes
                    + self.out_bytes + 1024) + (64 << 20) + 4 * self.B + 4096 + (4 * self.S * self.D + 4096 if rope != "off" else 0))
            free_b, total_b = hip.get_real_mem_info()
            allocator = SlabAllocator(hip, total_b, requested_pool_size=need)
            allocator.initialize()
        self.allocator = allocator
        A = allocator.allocate
        # Every layer's Q, then the kv offsets, in one allocation; every layer's output, then the
        # dispatcher's work words (ticket, status), in another: an end-to-end step is then one copy in
        # and one copy out, and the status word comes back with the results.
        self._q_tail = _round_up(self.L * self.q_bytes, 256)
        self._out_tail = _round_up(self.L * self.out_bytes, 256)
        self.q_all = A(self._q_tail + _round_up(4 * self.B, 256), "q_proj.output.all", MemoryRegion.ACTIVATIONS)
        self.out_all = A(self._out_tail + 256, "attention.output.all", MemoryRegion.ACTIVATIONS)
        self.offsets = types.SimpleNamespace(ptr=self.q_all.ptr + self._q_tail, size=4 * self.B)
        self.dispatcher = SplitKVAttentionDispatcher(
            hip, codegen, self.metadata, allocator=allocator, context_length=self.S, batch_size=self.B,
            num_splits=num_splits, fixed_chunk_size=fixed_chunk_size, compat=compat, min_chunk=min_chunk,
            output_f32=self.output_f32, strict_empty_splits=strict_empty_splits, emit_state=self.emit_state,
            prefetch_next_layer=prefetch_next_layer, fused_combine=fused_combine, variant=variant,
            fuse_rope=rope in ("fused", "fused-append"), fuse_append=(rope == "fused-append" or fuse_append), tensor_maps=tensor_maps,
            work_ptr=self.out_all.ptr + self._out_tail, balanced=balanced)

        self.k_cache = [A(self.kv_bytes, f"kv_cache.k.{i}", MemoryRegion.KV_CACHE) for i in range(self.n_kv)]
        self.v_cache = [A(self.kv_bytes, f"kv_cache.v.{i}", MemoryRegion.KV_CACHE) for i in range(self.n_kv)]
        # all layers' Q (and outputs) are contiguous so one copy moves a whole step's worth
        self.knew_all = A(self.L * self.kvnew_bytes, "k_proj.output.all", MemoryRegion.ACTIVATIONS)
        self.vnew_all = A(self.L * self.kvnew_bytes, "v_proj.output.all", MemoryRegion.ACTIVATIONS)

        self.tensor_mapping = {'kv_batch_stride_elements': self.kv_batch_stride}
        for l in range(self.L):
            self.tensor_mapping[f'blk.{l}.q_proj.output'] = self.q_all.ptr + l * self.q_bytes
            self.tensor_mapping[f'blk.{l}.k_proj.output'] = self.knew_all.ptr + l * self.kvnew_bytes
            self.tensor_mapping[f'blk.{l}.v_proj.output'] = self.vnew_all.ptr + l * self.kvnew_bytes
            self.tensor_mapping[f'blk.{l}.attention.output'] = self.out_all.ptr + l * self.out_bytes
            self.tensor_mapping[f'blk.{l}.kv_cache.k'] = self.k_cache[l % self.n_kv]
            self.tensor_mapping[f'blk.{l}.kv_cache.v'] = self.v_cache[l % self.n_kv]

        if self.rope != "off":
            from ..workloads import build_rope_cache
            rope_type = int(self.metadata.get('rope_type', 0))
            width = int(self.metadata.get('rotary_dim', self.D)) if rope_type == 2 else self.D
            cos, sin = build_rope_cache(self.S, width, float(rope_theta))
            self.rope_cos = A(cos.nbytes, "rope_cos", MemoryRegion.ACTIVATIONS)
            self.rope_sin = A(sin.nbytes, "rope_sin", MemoryRegion.ACTIVATIONS)
            hip.safe_memcpy_host_to_device(ctypes.c_void_p(self.rope_cos.ptr), cos, "rope_cos upload")
            hip.safe_memcpy_host_to_device(ctypes.c_void_p(self.rope_sin.ptr), sin, "rope_sin upload")
            self.tensor_mapping['rope_cos'] = self.rope_cos
            self.tensor_mapping['rope_sin'] = self.rope_sin

        # pinned staging: offsets, a step's Q, a step's outputs
        self._stage_q = hip.host_alloc(self._q_tail + _round_up(4 * self.B, 256))          # Q of every layer, then the offsets
        self._stage_offsets = ctypes.c_void_p(self._stage_q.value + self._q_tail)
        self._stage_out = hip.host_alloc(self._out_tail + 256)                               # outputs, then the work words
        ctypes.memset(self._stage_out.value, 0, self._out_tail + 256)
        self._graph_exec = None
        self._io_graph_exec = None      # staging copies + the layers' launches + the output copy, as one graph
        self._stage_event = None        # recorded after a step's staging copies; the next step waits for it
        self._stage_in_flight = False
        self.kernel_launches_per_step = 0

    # ---- data movement helpers ----------------------------------------------------
    def upload_layer(self, layer: int, q: np.ndarray, k_cache: Optional[np.ndarray] = None,
                     v_cache: Optional[np.ndarray] = None):
        """Host -> device of one layer's Q [B,Hq,D] and (optionally) its caches
        [B,max_seq,Hkv,D], all fp16."""
        self.hip.safe_memcpy_host_to_device(ctypes.c_void_p(self.q_all.ptr + layer * self.q_bytes),
                                            np.ascontiguousarray(q, dtype=np.float16), "q upload")
        if k_cache is not None:
            self.upload_cache(layer % self.n_kv, k_cache, v_cache)

    def upload_cache(self, buf: int, k_cache: np.ndarray, v_cache: np.ndarray):
        for dst, src in ((self.k_cache[buf], k_cache), (self.v_cache[buf], v_cache)):
            src = np.ascontiguousarray(src, dtype=np.float16)
            if src.shape != (self.B, self.S, self.Hkv, self.D):
                raise CudaSafetyError(f"cache shape {src.shape} != {(self.B, self.S, self.Hkv, self.D)}")
            self.hip.safe_memcpy_host_to_device(ctypes.c_void_p(dst.ptr), src, "kv upload")

    def upload_new_kv(self, layer: int, k_new: np.ndarray, v_new: np.ndarray):
        self.hip.safe_memcpy_host_to_device(ctypes.c_void_p(self.knew_all.ptr + layer * self.kvnew_bytes),
                                            np.ascontiguousarray(k_new, dtype=np.float16), "k_new upload")
        self.hip.safe_memcpy_host_to_device(ctypes.c_void_p(self.vnew_all.ptr + layer * self.kvnew_bytes),
                                            np.ascontiguousarray(v_new, dtype=np.float16), "v_new upload")

    def fill_cache_on_device(self, buf: int, seed: int, sigma: float = 1.0, outlier_prob: float = 0.0,
                             outlier_scale: float = 1.0):
        """Synthetic N(0, sigma) cache contents generated on the device."""
        n = self.B * self.kv_batch_stride
        self.hip.fill_normal_f16(ctypes.c_void_p(self.k_cache[buf].ptr), n, 2 * seed + 1, sigma, outlier_prob, outlier_scale)
        self.hip.fill_normal_f16(ctypes.c_void_p(self.v_cache[buf].ptr), n, 2 * seed + 2, sigma, outlier_prob, outlier_scale)

    def download_cache_rows(self, buf: int, b: int, n_rows: int):
        """(K, V) [n_rows, Hkv, D] fp16 of sequence b, for checking against the oracle."""
        row = self.Hkv * self.D
        k = np.empty((n_rows, self.Hkv, self.D), dtype=np.float16)
        v = np.empty_like(k)
        off = b * self.kv_batch_stride * 2
        self.hip.safe_memcpy_device_to_host(k, ctypes.c_void_p(self.k_cache[buf].ptr + off), "kv rows for output check")
        self.hip.safe_memcpy_device_to_host(v, ctypes.c_void_p(self.v_cache[buf].ptr + off), "kv rows for output check")
        assert k.nbytes == n_rows * row * 2
        return k, v

    # ---- graph ----------------------------------------------------------------------
    def _record_all(self):
        n = 0
        for l in range(self.L):
            launches = self.dispatcher.build_launches(l, self.tensor_mapping, self.offsets.ptr, batch=self.B)
            if not self.with_append and not self.dispatcher.fuse_append:
                launches = launches[1:]
            if self.launch_rewriter is not None:
                launches = self.launch_rewriter(l, launches)
            if self.rope == "separate":
                launches = [self.dispatcher.build_rope_launch(self.tensor_mapping, self.offsets.ptr, batch=self.B,
                                                              layer_idx=l)] + launches
            for fn, args, grid, block, smem in launches:
                self.hip.launch_kernel_recorded(fn, args, grid, block, smem)
                n += 1
            if self.per_layer_hook is not None:
                n += int(self.per_layer_hook(l) or 0)
        return n

    def build_decode_graph(self):
        """Capture all layers' launches once (hip_graph_executor.py:504-725)."""
        if self._graph_exec is not None:
            return
        self.hip.programmatic_launch = self.programmatic
        try:
            if not self.use_graph:
                n = len(self.dispatcher.build_launches(0, self.tensor_mapping, self.offsets.ptr, batch=self.B))
                n += 1 if self.rope == "separate" else 0
                self.kernel_launches_per_step = (n if (self.with_append or self.dispatcher.fuse_append) else n - 1) * self.L
                return
            self.hip.stream_begin_capture()
            try:
                self.kernel_launches_per_step = self._record_all()
            finally:
                graph = self.hip.stream_end_capture()
            self._graph_exec = self.hip.graph_instantiate(graph)
            self.hip.graph_destroy(graph)
        finally:
            self.hip.programmatic_launch = False

    def build_io_graph(self):
        """One graph for a whole end-to-end step: kv offsets and every layer's Q from pinned
        staging to the device, every layer's launches, every layer's output back to pinned
        staging.  A step is then one graph launch instead of three copies and a launch (the
        reference stages its offsets with a separate copy before each launch,
        vte/core/hip_graph_executor.py:772-789)."""
        if self._io_graph_exec is not None or not self.use_graph:
            return
        self.hip.programmatic_launch = self.programmatic
        try:
            self.hip.stream_begin_capture()
            try:
                self.hip.memcpy_h2d_async(ctypes.c_void_p(self.q_all.ptr), self._stage_q, self._q_tail + 4 * self.B,
                                          "q and kv offsets staging")
                self._record_all()
                self.hip.memcpy_d2h_async(self._stage_out, ctypes.c_void_p(self.out_all.ptr), self._out_tail + 16,
                                          "attention output and status word")
            finally:
                graph = self.hip.stream_end_capture()
            self._io_graph_exec = self.hip.graph_instantiate(graph)
            self.hip.graph_destroy(graph)
        finally:
            self.hip.programmatic_launch = False

    def _wait_for_staging(self):
        """The pinned staging buffers may be rewritten only after the previous step's asynchronous
        host-to-device copies have read them (a step enqueued with `read_output=False` returns
        before they ran)."""
        if self._stage_in_flight:
            self.hip.event_synchronize(self._stage_event)
            self._stage_in_flight = False

    def _mark_staging_copied(self):
        if self._stage_event is None:
            self._stage_event = self.hip.event_create()
        self.hip.event_record(self._stage_event)
        self._stage_in_flight = True

    def _update_staging_buffers(self, kv_offsets: np.ndarray):
        off = np.ascontiguousarray(kv_offsets, dtype=np.int32)
        if off.shape != (self.B,):
            raise CudaSafetyError(f"kv_offsets shape {off.shape} != ({self.B},)")
        if off.min() < 0 or off.max() >= self.S:
            raise CudaSafetyError(f"kv offset outside 0..{self.S - 1}")
        self._wait_for_staging()
        ctypes.memmove(self._stage_offsets.value, off.ctypes.data, off.nbytes)
        self.hip.memcpy_h2d_async(ctypes.c_void_p(self.offsets.ptr), self._stage_offsets, off.nbytes, "kv_offsets")
        self._mark_staging_copied()

    def launch_step(self):
        """Enqueue one decode step (no host synchronisation)."""
        if self._graph_exec is not None:
            self.hip.graph_launch(self._graph_exec)
        else:
            self.hip.programmatic_launch = self.programmatic
            try:
                self._record_all()
            finally:
                self.hip.programmatic_launch = False

    def execute_decode_batch(self, kv_offsets: np.ndarray, q_host: Optional[np.ndarray] = None,
                             read_output: bool = True) -> Optional[np.ndarray]:
        """One decode step end to end: stage offsets (and, when given, every layer's
        Q [L,B,Hq,D] fp16) host -> device, replay the graph, read every layer's
        output back.  Returns [L,B,Hq,D] (fp32 or fp16)."""
        self.build_decode_graph()
        nbytes = self.L * self.out_bytes
        if q_host is not None and read_output and self.use_graph:
            # the whole step as one graph launch
            self.build_io_graph()
            off = np.ascontiguousarray(kv_offsets, dtype=np.int32)
            if off.shape != (self.B,) or off.min() < 0 or off.max() >= self.S:
                raise CudaSafetyError(f"kv_offsets must be int32[{self.B}] within 0..{self.S - 1}")
            qh = np.ascontiguousarray(q_host, dtype=np.float16)
            if qh.nbytes != self.L * self.q_bytes:
                raise CudaSafetyError("q_host must be [L, B, Hq, D] fp16")
            self._wait_for_staging()
            ctypes.memmove(self._stage_offsets.value, off.ctypes.data, off.nbytes)
            ctypes.memmove(self._stage_q.value, qh.ctypes.data, qh.nbytes)
            self.hip.graph_launch(self._io_graph_exec)
            self.hip.stream_synchronize()
            # the status word travelled with the outputs: only a non-zero one needs the slow path
            if ctypes.c_int.from_address(self._stage_out.value + self._out_tail + 4).value != 0:
                self.dispatcher_check()
            return self._output_array(nbytes)
        else:
            self._update_staging_buffers(kv_offsets)
            if q_host is not None:
                qh = np.ascontiguousarray(q_host, dtype=np.float16)
                if qh.nbytes != self.L * self.q_bytes:
                    raise CudaSafetyError("q_host must be [L, B, Hq, D] fp16")
                # (_update_staging_buffers above already waited for the previous step's copies)
                ctypes.memmove(self._stage_q.value, qh.ctypes.data, qh.nbytes)
                self.hip.memcpy_h2d_async(ctypes.c_void_p(self.q_all.ptr), self._stage_q, qh.nbytes, "q staging")
                self._mark_staging_copied()
            self.launch_step()
            if not read_output:
                return None
            self.hip.memcpy_d2h_async(self._stage_out, ctypes.c_void_p(self.out_all.ptr), nbytes, "attention output")
            self.hip.stream_synchronize()
        self.dispatcher_check()
        return self._output_array(nbytes)

    def _output_array(self, nbytes: int) -> np.ndarray:
        dt = np.float32 if (self.output_f32 or self.emit_state) else np.float16
        flat = np.frombuffer((ctypes.c_char * nbytes).from_address(self._stage_out.value), dtype=dt)
        return flat.reshape(self.L, self.B, self.Hq, self.D + 2 if self.emit_state else self.D).copy()

    execute_decode = execute_decode_batch

    def dispatcher_check(self):
        """Raise if a split kernel reported a timed-out wait."""
        if self.dispatcher.work_ptr and hasattr(self.hip, "check_status"):
            self.hip.check_status(ctypes.c_void_p(self.dispatcher.work_ptr))

    def read_partials(self):
        """(partial_m, partial_l [B,Hq,C], partial_o [B,Hq,C,D]) of the last layer run."""
        pm, pl, po = self.dispatcher.partial_buffers
        C = self.dispatcher.max_chunks
        m = np.empty((self.B, self.Hq, C), dtype=np.float32)
        l = np.empty_like(m)
        o = np.empty((self.B, self.Hq, C, self.D), dtype=np.float32)
        self.hip.safe_memcpy_device_to_host(m, ctypes.c_void_p(pm.ptr), "partial output m")
        self.hip.safe_memcpy_device_to_host(l, ctypes.c_void_p(pl.ptr), "partial output l")
        self.hip.safe_memcpy_device_to_host(o, ctypes.c_void_p(po.ptr), "partial output o")
        return m, l, o

    def cleanup(self):
        if self._stage_event is not None:
            self.hip.event_destroy(self._stage_event)
            self._stage_event = None
            self._stage_in_flight = False
        if self._graph_exec is not None:
            self.hip.graph_exec_destroy(self._graph_exec)
            self._graph_exec = None
        if self._io_graph_exec is not None:
            self.hip.graph_exec_destroy(self._io_graph_exec)
            self._io_graph_exec = None
        for p in (self._stage_q, self._stage_out):
            if p is not None and p.value:
                self.hip.host_free(p)
        self._stage_offsets = self._stage_q = self._stage_out = None
        if self._owns_allocator:
            self.allocator.cleanup()
