"""Split-KV (flash-decoding) attention dispatcher for decode (one query token).

Drop-in for `SplitKVAttentionDispatcher` of vte/core/split_kv_attention.py:52-229:
same constructor arguments, same `.enabled` switch (`VTE_DISABLE_ATTN_SPLITKV`),
same `build_launches(layer_idx, tensor_mapping, kv_offset_ptr, batch, q_name,
k_name, v_name)` returning three `(function, args, grid, block, shared_mem)`
tuples (append, partial, reduce; append and one launch with `fused_combine=True`) that an executor records with
`launch_kernel_recorded`, same scratch policy (one set of partial buffers shared
by all layers, :114-128), same tensor-name resolution (:72-98, :166-176).

What differs is what the tuples launch.  By default the partial launch is the
persistent sm_100a kernel (`vteb_split_kv_partial_d*_kernel`, grid = one CTA per
SM) and the reduce launch is `vteb_split_kv_combine_*`; `compat=True` (or
`VTE_B200_COMPAT_KERNELS=1`) emits the reference-named kernels with the
reference's own grids instead.  `max_chunks` is a split COUNT unless
`fixed_chunk_size` is given, in which case the reference's arithmetic
(`max_chunks = ceil(context_length / chunk_size)`, :61-62) is used and the
kernels are compiled with that chunk length.
"""
from __future__ import annotations

import ctypes
import math
import os

from ..bridge.errors import CudaSafetyError
from ..bridge.memory import MemoryRegion
from ..config import ENV_COMPAT_KERNELS, ENV_DISABLE_SPLITKV

SPLIT_KV_CHUNK_SIZE = 32          # the reference's historical chunk (RX 7600, 32 CUs)
MAX_SPLITS = 256
TARGET_CHUNK_POSITIONS = 512      # smallest chunk length aimed at when many sequences share the GPU
FLAG_WRITE_EMPTY_O = 1
FLAG_DIRECT_OUTPUT = 2
FLAG_TENSOR_MAPS = 4
FLAG_PREFETCH_Q = 8
FLAG_BALANCED = 16
COMPACT_MAX_CONTEXT = 262144      # one sequence up to this long: the compact CTA shape (launches of tens of microseconds)
SHORT_CONTEXT_MAX = 2048          # one sequence up to this many positions: at most 32 splits (see choose_split_count)
UNSPLIT_MAX_CONTEXT = 128         # below this, one CTA per (sequence, head group) finishes before a combine could launch


def _chunk_size_for_cus(num_cus: int) -> int:
    """The reference's rule (vte/core/split_kv_attention.py:40-49): 1024 / CUs,
    rounded, kept within [8, 64]; 32 when the count is unknown."""
    if num_cus <= 0:
        return SPLIT_KV_CHUNK_SIZE
    return max(8, min(64, round(1024 / num_cus)))


def choose_chunk_positions(num_sms: int, batch: int, n_hgroups: int, context_length: int) -> int:
    """Positions per split aimed at when several sequences share the GPU: about four work items per
    SM if every sequence were half the configured context, as a power of two within [512, 2048].
    Measured on B200: a work item costs a few microseconds of fixed time (its Q rows, the cross-warp
    merge, the ragged last tile), which outweighs the better balance of small items.  Per layer, with
    256 / 512 / 1024 / 2048-position items: the 64-sequence ragged batch of 8 x 64-wide heads
    - / - / 191 / 203 us, its 16-sequence share 61.4 / 60.4 / 62.2 / 71.2 us, its 8-sequence share
    37.7 / 34.8 / 39.2 / - us; two sequences of 2 x 256-wide heads 36.9 / 32.0 / 35.7 / - us, sixteen
    - / - / 208 / 201 us."""
    est_positions = batch * n_hgroups * max(1, context_length // 2)
    target = est_positions / max(1, num_sms * 4)
    chunk = TARGET_CHUNK_POSITIONS
    while chunk < target and chunk < 2048:
        chunk *= 2
    return chunk


def balanced_split_count(num_sms: int, batch: int, n_hgroups: int) -> int:
    """Splits reserved per (sequence, head group) for the balanced partition.  A pair of S positions is
    cut into at most ceil(S / share) + 1 pieces, where share = all positions / num_sms; with equal
    lengths that is num_sms / pairs + 1.  Eight times that (one pair may be eight times the mean length
    before the kernel has to enlarge the shares and leave CTAs idle), kept within the 64 splits of the
    one-warp-per-row combine, whose cost follows the splits in use and not the splits reserved; with so
    few pairs that 64 cannot hold 2.5 times the mean, that many and the wide combine."""
    pairs = max(1, batch * n_hgroups)
    want = math.ceil(8 * num_sms / pairs) + 1
    if want <= 64:
        return max(8, want)
    need = min(num_sms, math.ceil(2.5 * num_sms / pairs)) + 1
    return 64 if need <= 64 else min(MAX_SPLITS, need)


def balanced_pieces(lengths, n_hgroups: int, n_ctas: int, max_chunks: int, tile: int):
    """Host restatement of the split kernel's balanced partition (split_kv_fast.cuh, BalancedShare):
    the list, per CTA, of its pieces (sequence, head group, split index, first position, end position).
    Used by tests and for sizing; the kernel derives the same cuts from the offsets on the device."""
    lengths = [int(x) for x in lengths]
    total = sum(lengths) * n_hgroups
    per = -(-total // n_ctas)
    slots = max(1, max_chunks - 1)
    per = max(per, -(-max(lengths) // slots), 1)
    per = -(-per // tile) * tile
    firsts, acc = [], 0
    for s in lengths:
        for h in range(n_hgroups):
            firsts.append((acc, s, len(firsts) // n_hgroups, h))
            acc += s
    out = []
    for cta in range(n_ctas):
        lo, hi = min(cta * per, total), min((cta + 1) * per, total)
        mine = []
        for first, s, b, h in firsts:
            a, e = max(lo, first), min(hi, first + s)
            if e > a:
                mine.append((b, h, a // per - first // per, a - first, e - first))
        out.append(mine)
    return out


def choose_split_count(num_sms: int, batch: int, n_hgroups: int, context_length: int) -> int:
    """Split count when the caller does not fix one.

    One sequence: as many splits as SMs, so the persistent grid is exactly one
    wave of equal work items.  Several sequences: chunks of
    `choose_chunk_positions` (capped at 256 splits for the longest context), so
    that ragged lengths balance through the work queue while the fp32 partials
    stay a few percent of the K/V bytes.
    """
    if context_length <= UNSPLIT_MAX_CONTEXT:
        return 1                                   # unsplit: the split launch stores the output itself
    # One sequence: a split per SM for a long context; up to SHORT_CONTEXT_MAX positions at most 32 splits
    # (and never more than the context has 16-position blocks), which the compact shape pairs with the
    # small combine (one L2 round trip for up to 32 splits).  Per layer, 28 layers per graph, 32 splits +
    # small combine against a split per block or SM + wide combine: 512 positions 4.89 / 5.48 us, 768:
    # 5.12 / 5.55, 1,024: 5.19 / 5.57, 1,536: 5.54 / 5.82, 2,048: 5.83 / 5.92, 3,000: 6.33 / 6.28,
    # 4,096: 6.84 / 6.33.
    blocks = max(1, -(-context_length // 16))
    short = 32 if context_length <= SHORT_CONTEXT_MAX else MAX_SPLITS
    if batch * n_hgroups <= 1:
        return max(1, min(MAX_SPLITS, num_sms, blocks, short))
    if batch == 1:
        return max(1, min(MAX_SPLITS, num_sms // n_hgroups, blocks, short))
    chunk = choose_chunk_positions(num_sms, batch, n_hgroups, context_length)
    return max(1, min(MAX_SPLITS, math.ceil(context_length / chunk)))


class SplitKVAttentionDispatcher:
    def __init__(self, hip, codegen, metadata: dict, allocator=None, context_length: int = 4096,
                 batch_size: int = 1, *, num_splits: int | None = None, fixed_chunk_size=None,
                 compat: bool | None = None, min_chunk: int | None = None, output_f32: bool = False,
                 strict_empty_splits: bool = False, emit_state: bool = False, prefetch_next_layer: bool = True,
                 fused_combine: bool | None = None, variant: str = "auto", fuse_rope: bool = False,
                 tensor_maps: bool = True, work_ptr: int | None = None, fuse_append: bool = False,
                 balanced: bool | None = None):
        self.hip = hip
        self.codegen = codegen
        self.metadata = metadata or {}
        self.allocator = allocator
        self.batch_size = int(batch_size)
        self.context_length = int(context_length)
        self.output_f32 = bool(output_f32)
        self.strict_empty_splits = bool(strict_empty_splits)
        # emit_state: the reduce launch writes one unnormalised (o[D], m, l) row per query head
        # instead of the attention output; used when the KV range is sharded across GPUs
        self.emit_state = bool(emit_state)
        # hand the split kernel the next layer's caches so its loaders can pull them into L2
        self.prefetch_next_layer = bool(prefetch_next_layer)
        self.compat = bool(os.environ.get(ENV_COMPAT_KERNELS)) if compat is None else bool(compat)

        self.num_q_heads = int(self.metadata.get('attention.head_count', 12))
        self.num_kv_heads = int(self.metadata.get('attention.head_count_kv', 2))
        self.head_dim = int(self.metadata.get('attention.key_length', 128))
        num_cus = hip.get_num_cus() if hip is not None and hasattr(hip, 'get_num_cus') else 32
        self.num_sms = num_cus

        # CTA shape of the split kernel.  "full": 8 consumer + 2 loader warps.  "compact": 6 + 2
        # warps of at most 160 registers, which leaves register-file room on every SM for the combine
        # launch's CTAs to sit beside the split CTA, so the combine starts the moment the split ends
        # and the launch after it is not held back.  Measured on B200, 32k context, one sequence:
        # 10.6 us per layer compact against 12.5 us full; batches of ragged sequences and a
        # one-million-position sequence run a few percent slower compact (fewer consumer warps do not
        # keep up with a stream that lasts hundreds of microseconds).  "auto" therefore takes compact
        # for one sequence of up to COMPACT_MAX_CONTEXT positions and full otherwise.
        if variant not in ("full", "compact", "auto"):
            raise CudaSafetyError(f"variant must be full, compact or auto, not {variant!r}")
        self._plan = None
        self.compact = False
        if hip is not None and hasattr(hip, 'split_kv_plan'):
            self._plan = hip.split_kv_plan(self.num_q_heads, self.num_kv_heads, self.head_dim)
            want_compact = variant == "compact" or (variant == "auto" and self.batch_size == 1
                                                    and self.context_length <= COMPACT_MAX_CONTEXT
                                                    and not fused_combine)
            if want_compact and not self.compat:
                compact_plan = hip.split_kv_plan(self.num_q_heads, self.num_kv_heads, self.head_dim, compact=True)
                if compact_plan.ok:
                    self._plan, self.compact = compact_plan, True
        if self.emit_state and (self.compat or self._plan is None or not self._plan.ok):
            raise CudaSafetyError("emit_state needs the fast kernels (group <= 8, head_dim 64/128/256)")
        if not self.compat and (self._plan is None or not self._plan.ok):
            # geometry outside the fast kernel (group > 8, unusual head_dim): reference-geometry kernels
            self.compat = True

        # fused_combine: the split launch also merges the splits (after a grid-wide barrier), so a
        # layer is append + ONE launch.  Needs all eight consumer warps (hg divides 8).
        can_fuse = ((not self.compat) and (not self.compact) and self._plan is not None and self._plan.ok
                    and 8 % self._plan.hg == 0)
        # Measured on B200 at 32k context: 15.1 us per layer fused against 13.4 us with the separate
        # combine launch (the grid barrier costs more than the launch it saves), so it is opt-in.
        self.fused_combine = bool(fused_combine) and can_fuse

        if fixed_chunk_size is not None:
            self.chunk_size = _chunk_size_for_cus(num_cus) if fixed_chunk_size == "auto" else int(fixed_chunk_size)
            if self.chunk_size <= 0:
                raise CudaSafetyError(f"fixed_chunk_size must be positive, got {fixed_chunk_size}")
            self.max_chunks = max(1, math.ceil(self.context_length / self.chunk_size))
            self.fixed_chunk = True
            self.balanced = False
            if balanced:
                raise CudaSafetyError("the balanced partition and a fixed chunk size exclude each other")
        else:
            self.fixed_chunk = False
            n_hg = self._plan.n_hgroups if (self._plan is not None and self._plan.ok) else self.num_kv_heads
            # balanced: every CTA takes an equal share of all cached positions instead of drawing
            # fixed-size splits from a work queue (split_kv_fast.cuh, BalancedShare).  Chosen when several
            # sequences share the GPU and the caller fixed neither the split count nor a minimum split.
            fast = (not self.compat) and self._plan is not None and self._plan.ok
            auto_count = not num_splits
            self.balanced = fast and not self.fused_combine and not self.compact and (
                (balanced is None and auto_count and min_chunk is None and self.batch_size > 1
                 and self.context_length > UNSPLIT_MAX_CONTEXT) or bool(balanced))
            if self.balanced and self.batch_size * n_hg < 2:
                self.balanced = False
            if num_splits:
                self.max_chunks = int(num_splits)
            elif self.balanced:
                self.max_chunks = balanced_split_count(num_cus, self.batch_size, n_hg)
            else:
                self.max_chunks = choose_split_count(num_cus, self.batch_size, n_hg, self.context_length)
            if self.balanced and self.max_chunks < 2:
                raise CudaSafetyError("the balanced partition needs at least two splits")
            if not (1 <= self.max_chunks <= 65535):
                raise CudaSafetyError(f"split count {self.max_chunks} outside 1..65535")
            self.chunk_size = 0
        if min_chunk is None:
            n_hg = self._plan.n_hgroups if (self._plan is not None and self._plan.ok) else self.num_kv_heads
            min_chunk = (choose_chunk_positions(num_cus, self.batch_size, n_hg, self.context_length)
                         if (self.batch_size > 1 and not self.fixed_chunk and not self.balanced) else 0)
        self.min_chunk = int(min_chunk)

        # fuse_rope: q_name / k_name are the UN-rotated projections; the append launch rotates the K
        # row as it enters the cache and the split launch rotates Q as it loads it, which removes the
        # standalone rotation launch from the layer.  Tables come from tensor_mapping['rope_cos'] /
        # ['rope_sin'] (vte/core/kernel_arg_builder.py:394-395), type and width from the metadata keys
        # `rope_type` / `rotary_dim` (:401-406).  The reference tried this fusion and took it out again
        # (docs/PERFORMANCE.md, "RoPE fusion into Split-KV attention").
        # fuse_append: no append launch at all; the split kernel's CTA whose tile holds a sequence's newest
        # position writes the new K row (rotated when fuse_rope) and V row into the cache and into its
        # tile.  A layer is then split + combine.  Uses the rotating kernels (rotation type -1 = none).
        self.fuse_append = bool(fuse_append)
        self.fuse_rope = bool(fuse_rope)
        self.rope_type = int(self.metadata.get('rope_type', 0))
        self.rotary_dim = int(self.metadata.get('rotary_dim', self.head_dim))
        if self.fuse_append and self.compat:
            raise CudaSafetyError("fuse_append needs the fast kernels")
        if self.fuse_rope:
            if self.compat:
                raise CudaSafetyError("fuse_rope needs the fast kernels")
            if self.rope_type not in (0, 1, 2):
                raise CudaSafetyError(f"rope_type {self.rope_type} not in 0, 1, 2")
            if self.rope_type == 2 and (self.rotary_dim not in (32, 64, 128, 256) or self.rotary_dim > self.head_dim):
                raise CudaSafetyError(f"rotary_dim {self.rotary_dim} must be 32, 64, 128 or 256 and at most head_dim")

        # tensor_maps: whole K/V tiles are fetched with tensor-map (TMA) box copies; ragged ends and
        # caches whose sequence stride is not a whole number of position rows use 16-byte copies
        self.tensor_maps = bool(tensor_maps) and hip is not None and hasattr(hip, 'kv_tensor_map')
        self._tensor_map_cache = {}

        # work_ptr: 16 bytes of device memory for the work words (ticket, status) supplied by the
        # caller, e.g. next to its output buffer so that one copy brings the status word back with the
        # results; by default they come from the allocator with the other scratch
        self._external_work_ptr = int(work_ptr) if work_ptr else None

        self._kernel_cache = {}
        self._rows_combine = False
        self._small_combine = False
        self._partial_m = self._partial_l = self._partial_o = self._work = None
        self.enabled = not bool(os.environ.get(ENV_DISABLE_SPLITKV)) and allocator is not None

    @property
    def split_kernel_name(self) -> str:
        """Symbol of the fast split kernel this dispatcher launches.  `compact_cs`: splits of one
        16-position block (a context of up to 16 positions per SM) in the compact kernel for 128-wide heads
        with three warps per KV head: the head's warps split the output columns instead of the blocks and
        the item ends without a cross-warp merge.  Measured per layer, 28 layers per graph, column split
        against the ordinary compact kernel: 512 positions 5.62 / 5.85 us, 1,024: 5.79 / 6.13, 2,048:
        5.88 / 6.37, 4,096 (two blocks per split): 6.42 / 6.35, 8,192: 7.59 / 7.09, 16,384: 9.67 / 8.34:
        from two blocks on, the repeated score computation costs more than the merge."""
        rotating = self.fuse_rope or self.fuse_append
        longest_split = -(-self.context_length // max(1, self.max_chunks))
        column_split = (self.compact and not rotating and self.head_dim == 128 and self._plan.hg == 2
                        and self.max_chunks > 1 and longest_split <= 16)
        return (f"vteb_split_kv_partial_{'compact_' if self.compact else ''}{'cs_' if column_split else ''}"
                f"{'rope_' if rotating else ''}d{self.head_dim}_kernel")

    # -- tensor-name resolution -------------------------------------------------
    @staticmethod
    def _resolve_ptr(tensor_mapping: dict, name: str) -> int:
        p = tensor_mapping.get(name)
        if p is None:
            return 0
        return int(p.ptr) if hasattr(p, 'ptr') else int(p)

    def _resolve_kv_cache_ptrs(self, layer_idx: int, tensor_mapping: dict):
        """`blk.{l}.kv_cache.k/.v`, then `kv_cache.layer_{l}.k/.v`, then the pooled
        layout (per layer: K block, then V block, each
        batch * Hkv * D * 2 * context_length bytes; vte/compiler/qwen_mapper.py:321-351)."""
        def get(*names):
            for n in names:
                p = tensor_mapping.get(n)
                if p is not None:
                    return int(p.ptr) if hasattr(p, 'ptr') else int(p)
            return None
        k_ptr = get(f'blk.{layer_idx}.kv_cache.k', f'kv_cache.layer_{layer_idx}.k')
        v_ptr = get(f'blk.{layer_idx}.kv_cache.v', f'kv_cache.layer_{layer_idx}.v')
        if k_ptr is None or v_ptr is None:
            pool = get('KV Cache Pool')
            if pool is not None:
                half = self.batch_size * self.num_kv_heads * self.head_dim * 2 * self.context_length
                k_ptr = pool + layer_idx * 2 * half
                v_ptr = k_ptr + half
        return int(k_ptr or 0), int(v_ptr or 0)

    # -- kernels and scratch ------------------------------------------------------
    def _get_kernels(self):
        if 'append' not in self._kernel_cache:
            arch = self.hip.get_gpu_architecture()
            params = {'split_kv_chunk_size': self.chunk_size} if self.fixed_chunk else {}
            load = lambda template, symbol: self.codegen.load_kernel_safe(self.hip, template, arch, symbol, **params)[1]
            self._kernel_cache['append'] = load(
                'kv_cache_append', 'kv_cache_append_rope_kernel' if self.fuse_rope else 'kv_cache_append_kernel')
            if self.compat:
                self._kernel_cache['partial'] = load('flash_attention_split_kv_partial',
                                                     'flash_attention_split_kv_partial_kernel')
                self._kernel_cache['reduce'] = load(
                    'flash_attention_split_kv_reduce',
                    'flash_attention_split_kv_reduce_f32_kernel' if self.output_f32
                    else 'flash_attention_split_kv_reduce_kernel')
            else:
                self._kernel_cache['partial'] = load('decode_attention', self.split_kernel_name)
                # short split lists (batched decode): one warp per (sequence, head) row;
                # long ones (one sequence spread over every SM): one CTA per 32 columns
                # The compact split kernel needs a combine whose CTAs sit beside its own: the wide combine
                # (76 registers) or, up to 32 splits, the small one (one warp per 32 columns of a head, every
                # load in flight at once, 64 registers); the row kernel (111 registers) would start only when
                # the split CTA has left (512-position context with 32 splits, per layer: 7.26 us with the row
                # kernel, 5.44 with the wide combine).
                self._small_combine = self.max_chunks <= 32 and self.compact
                self._rows_combine = self.max_chunks <= 64 and not self.compact
                self._kernel_cache['reduce'] = load(
                    'decode_attention',
                    'vteb_split_kv_combine_small_kernel' if self._small_combine else
                    'vteb_split_kv_combine_rows_kernel' if self._rows_combine else
                    'vteb_split_kv_combine_state_kernel' if self.emit_state else
                    'vteb_split_kv_combine_f32_kernel' if self.output_f32 else 'vteb_split_kv_combine_f16_kernel')

            # One scratch set shared by every layer: layers run strictly one after
            # another inside a decode step, so rewriting the same buffers is safe.
            stats_size = self.batch_size * self.num_q_heads * self.max_chunks * 4
            o_size = stats_size * self.head_dim
            self._partial_m = self.allocator.allocate(stats_size, "attn_splitkv_m", MemoryRegion.SCRATCH)
            self._partial_l = self.allocator.allocate(stats_size, "attn_splitkv_l", MemoryRegion.SCRATCH)
            self._partial_o = self.allocator.allocate(o_size, "attn_splitkv_o", MemoryRegion.SCRATCH)
            # work[0]: work-queue ticket (zero between launches), work[1]: status word
            if self._external_work_ptr is not None:
                import types
                self._work = types.SimpleNamespace(ptr=self._external_work_ptr, size=16)
            else:
                self._work = self.allocator.allocate(16, "attn_splitkv_work", MemoryRegion.SCRATCH)
            if hasattr(self.hip, 'safe_memset'):
                self.hip.safe_memset(ctypes.c_void_p(self._work.ptr), 16, "attn_splitkv_work")
        return self._kernel_cache['append'], self._kernel_cache['partial'], self._kernel_cache['reduce']

    def build_rope_launch(self, tensor_mapping: dict, kv_offset_ptr: int, batch: int = 1,
                          q_name: str = None, k_name: str = None, layer_idx: int = 0, block_size: int = 256):
        """The standalone rotation launch of one decode step, for callers that keep it separate:
        `rope_kernel` with the reference's eleven arguments (vte/core/kernel_arg_builder.py:388-431)
        and its grid rule (ceil(elements of Q / block) blocks in x, batch in y;
        vte/core/hip_graph_executor.py:359-367).  Rotates Q and K in place."""
        arch = self.hip.get_gpu_architecture()
        if 'rope' not in self._kernel_cache:
            self._kernel_cache['rope'] = self.codegen.load_kernel_safe(self.hip, 'rope', arch, 'rope_kernel')[1]
        q_ptr = self._resolve_ptr(tensor_mapping, q_name or f'blk.{layer_idx}.q_proj.output')
        k_ptr = self._resolve_ptr(tensor_mapping, k_name or f'blk.{layer_idx}.k_proj.output')
        cos_ptr = self._resolve_ptr(tensor_mapping, 'rope_cos')
        sin_ptr = self._resolve_ptr(tensor_mapping, 'rope_sin')
        kv_offset_ptr = int(kv_offset_ptr.value or 0) if isinstance(kv_offset_ptr, ctypes.c_void_p) else int(kv_offset_ptr or 0)
        for name, p in (("q", q_ptr), ("k", k_ptr), ("rope_cos", cos_ptr), ("rope_sin", sin_ptr), ("kv offsets", kv_offset_ptr)):
            if not p:
                raise CudaSafetyError(f"{name} pointer could not be resolved (null)")
        vp, ci = ctypes.c_void_p, ctypes.c_int
        args = [vp(q_ptr), vp(k_ptr), vp(cos_ptr), vp(sin_ptr), ci(1), ci(self.num_q_heads), ci(self.num_kv_heads),
                ci(self.head_dim), vp(kv_offset_ptr), ci(self.rope_type), ci(self.rotary_dim)]
        grid_x = max(1, -(-(self.num_q_heads * self.head_dim) // block_size))
        return (self._kernel_cache['rope'], args, (grid_x, batch, 1), (block_size, 1, 1), 0)

    @property
    def work_ptr(self) -> int:
        return self._work.ptr if self._work is not None else 0

    @property
    def partial_buffers(self):
        return self._partial_m, self._partial_l, self._partial_o

    # -- tensor maps ----------------------------------------------------------------
    @staticmethod
    def _null_tensor_map():
        from ..bridge.cuda_runtime import KvTensorMap
        return KvTensorMap()

    def _tensor_maps_for(self, k_cache_ptr: int, v_cache_ptr: int, kv_batch_stride: int, batch: int):
        """(K map, V map) for one layer's caches, or (None, None) when tensor-map copies do not apply."""
        row_halves = self.num_kv_heads * self.head_dim
        if not self.tensor_maps or row_halves % 64 or kv_batch_stride % row_halves:
            return None, None
        rows_per_seq = kv_batch_stride // row_halves if kv_batch_stride else self.context_length
        n_rows = max(1, rows_per_seq * max(1, batch))
        key = (k_cache_ptr, v_cache_ptr, n_rows)
        if key not in self._tensor_map_cache:
            self._tensor_map_cache[key] = (self.hip.kv_tensor_map(k_cache_ptr, n_rows, row_halves, self._plan.tile),
                                           self.hip.kv_tensor_map(v_cache_ptr, n_rows, row_halves, self._plan.tile))
        return self._tensor_map_cache[key]

    # -- launches -----------------------------------------------------------------
    def _validate(self, batch, q_ptr, k_cache_ptr, v_cache_ptr, output_ptr, kv_offset_ptr, kv_batch_stride):
        if batch <= 0 or batch > self.batch_size:
            raise CudaSafetyError(f"batch {batch} outside 1..{self.batch_size} (scratch is sized for batch_size)")
        for name, p in (("q", q_ptr), ("k_cache", k_cache_ptr), ("v_cache", v_cache_ptr),
                        ("attention output", output_ptr), ("kv offsets", kv_offset_ptr)):
            if not p:
                raise CudaSafetyError(f"{name} pointer could not be resolved (null)")
        for name, p in (("q", q_ptr), ("k_cache", k_cache_ptr), ("v_cache", v_cache_ptr)):
            if p % 16:
                raise CudaSafetyError(f"{name} pointer 0x{p:X} is not 16-byte aligned")
        if self.head_dim not in (64, 128, 256):
            raise CudaSafetyError(f"head_dim {self.head_dim} not supported (64, 128, 256)")
        if self.num_q_heads % self.num_kv_heads:
            raise CudaSafetyError(f"{self.num_q_heads} query heads are not a multiple of {self.num_kv_heads} KV heads")
        if kv_batch_stride < 0 or kv_batch_stride >= 2 ** 31:
            raise CudaSafetyError(f"kv_batch_stride_elements {kv_batch_stride} does not fit the kernel's int argument")
        if kv_batch_stride % 8:
            raise CudaSafetyError(f"kv_batch_stride_elements {kv_batch_stride} must be a multiple of 8")
        if batch > 1 and kv_batch_stride == 0:
            raise CudaSafetyError("kv_batch_stride_elements is 0 with batch > 1: sequences would alias")

    def build_launches(self, layer_idx: int, tensor_mapping: dict, kv_offset_ptr: int, batch: int = 1,
                       q_name: str = None, k_name: str = None, v_name: str = None):
        """[(append_fn, args, grid, block, smem), (partial_fn, ...), (reduce_fn, ...)]
        for one layer.  Names default to the reference's convention
        (`blk.{l}.q_proj.output` etc.); pass the graph node's real input names
        when RoPE or a per-head norm writes elsewhere."""
        append_fn, partial_fn, reduce_fn = self._get_kernels()
        Hq, Hkv, D, C = self.num_q_heads, self.num_kv_heads, self.head_dim, self.max_chunks
        attention_scale = self.metadata.get('attention_scale')
        scale = float(attention_scale) if attention_scale else 1.0 / math.sqrt(D)

        q_ptr = self._resolve_ptr(tensor_mapping, q_name or f'blk.{layer_idx}.q_proj.output')
        k_proj_ptr = self._resolve_ptr(tensor_mapping, k_name or f'blk.{layer_idx}.k_proj.output')
        v_proj_ptr = self._resolve_ptr(tensor_mapping, v_name or f'blk.{layer_idx}.v_proj.output')
        output_ptr = self._resolve_ptr(tensor_mapping, f'blk.{layer_idx}.attention.output')
        k_cache_ptr, v_cache_ptr = self._resolve_kv_cache_ptrs(layer_idx, tensor_mapping)
        kv_batch_stride = int(tensor_mapping.get('kv_batch_stride_elements', 0))
        kv_offset_ptr = int(kv_offset_ptr.value or 0) if isinstance(kv_offset_ptr, ctypes.c_void_p) else int(kv_offset_ptr or 0)
        self._validate(batch, q_ptr, k_cache_ptr, v_cache_ptr, output_ptr, kv_offset_ptr, kv_batch_stride)

        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        append_args = [vp(k_proj_ptr), vp(v_proj_ptr), vp(k_cache_ptr), vp(v_cache_ptr),
                       ci(Hkv), ci(D), vp(kv_offset_ptr), ci(kv_batch_stride)]
        rope_tail = []
        if self.fuse_rope:
            cos_ptr = self._resolve_ptr(tensor_mapping, 'rope_cos')
            sin_ptr = self._resolve_ptr(tensor_mapping, 'rope_sin')
            if not cos_ptr or not sin_ptr or cos_ptr % 4 or sin_ptr % 4:
                raise CudaSafetyError("fuse_rope: rope_cos / rope_sin missing from the tensor mapping or misaligned")
            rope_tail = [vp(cos_ptr), vp(sin_ptr), ci(self.rope_type), ci(self.rotary_dim)]
        append = (append_fn, append_args + rope_tail, (batch, Hkv, 1), (D, 1, 1), 0)
        split_tail = list(rope_tail)
        if self.fuse_rope or self.fuse_append:
            if not self.fuse_rope:
                split_tail = [vp(0), vp(0), ci(-1), ci(0)]                 # rotation type -1: none
            # the kernel reads the new rows with 16-byte asynchronous copies (they fill the masked rows of
            # the sequence's last tile), so they need the same alignment as q and the caches
            if self.fuse_append and (not k_proj_ptr or not v_proj_ptr or k_proj_ptr % 16 or v_proj_ptr % 16):
                raise CudaSafetyError("fuse_append: the new K / V rows could not be resolved or are not 16-byte aligned")
            split_tail += [vp(k_proj_ptr if self.fuse_append else 0), vp(v_proj_ptr if self.fuse_append else 0)]

        reference_partial_args = [
            vp(q_ptr), vp(k_cache_ptr), vp(v_cache_ptr),
            vp(self._partial_m.ptr), vp(self._partial_l.ptr), vp(self._partial_o.ptr),
            ci(Hq), ci(Hkv), ci(D), cf(scale), vp(kv_offset_ptr), ci(kv_batch_stride), ci(C)]
        reduce_args = [vp(self._partial_m.ptr), vp(self._partial_l.ptr), vp(self._partial_o.ptr),
                       vp(output_ptr), ci(Hq), ci(D), ci(C)]

        if self.compat:
            partial = (partial_fn, reference_partial_args, (batch, Hq, C), (D, 1, 1), 2 * D * 4)
            reduce = (reduce_fn, reduce_args, (batch, Hq, 1), (D, 1, 1), C * 4)
            return [append, partial, reduce]

        plan = self._plan
        items = batch * plan.n_hgroups * C
        n_ctas = self.num_sms if self.balanced else max(1, min(items, self.num_sms))
        flags = FLAG_WRITE_EMPTY_O if self.strict_empty_splits else 0
        if self.balanced:
            flags |= FLAG_BALANCED
        # Under programmatic dependent launch the split CTAs start while the launch before them still runs:
        # the loader asks L2 for the Q rows (a hint only, no data reaches the SM) so that the consumers'
        # fetch after the dependency wait does not go to DRAM.  With plain stream order the wait returns at
        # once and the consumers' own loads would queue behind the prefetch (measured: 9.66 -> 9.81 us per
        # launch in a graph of split launches only), so the flag is left off.
        if getattr(self.hip, 'programmatic_launch', False):
            flags |= FLAG_PREFETCH_Q
        next_k = next_v = 0
        if self.prefetch_next_layer:
            next_k, next_v = self._resolve_kv_cache_ptrs(layer_idx + 1, {k: v for k, v in tensor_mapping.items()
                                                                         if k != 'KV Cache Pool'})
            if not (next_k and next_v) or next_k % 16 or next_v % 16:
                next_k = next_v = 0
        out_kind = 3 if self.emit_state else (2 if self.output_f32 else 1)
        # One split and an ordinary output: the split launch normalises and stores the attention
        # output itself (the reference's unsplit kernel, flash_attention.hip.template:29-113, in one
        # launch).  Needs one CTA per work item, because nothing resets the work queue afterwards.
        direct = C == 1 and not self.emit_state and not self.strict_empty_splits and items <= self.num_sms
        if direct:
            flags |= FLAG_DIRECT_OUTPUT
        pass_output = self.fused_combine or direct
        tmap_k, tmap_v = self._tensor_maps_for(k_cache_ptr, v_cache_ptr, kv_batch_stride, batch)
        if tmap_k is not None:
            flags |= FLAG_TENSOR_MAPS
        else:
            tmap_k, tmap_v = self._null_tensor_map(), self._null_tensor_map()
        partial_args = reference_partial_args + [
            ci(batch), ci(self.min_chunk), ci(flags), vp(0), vp(self._work.ptr), vp(self._work.ptr + 4),
            vp(next_k), vp(next_v),
            vp(output_ptr if pass_output else 0), ci(out_kind if pass_output else 0), tmap_k, tmap_v] + split_tail
        partial = (partial_fn, partial_args, (n_ctas, 1, 1), (plan.threads, 1, 1), plan.smem_bytes)
        head = [] if self.fuse_append else [append]
        if self.fused_combine or direct:
            return head + [partial]
        if self._small_combine:
            rows = batch * Hq
            units = rows * (D // 32)
            combine_args = reduce_args + [ci(out_kind), vp(self._work.ptr), ci(rows), ci(1)]
            return head + [partial, (reduce_fn, combine_args, ((units + 7) // 8, 1, 1), (256, 1, 1), 0)]
        if self._rows_combine:
            rows = batch * Hq
            epl = self.hip.combine_rows_epl(rows, D)
            units = rows * (D // (32 * epl))
            combine_args = reduce_args + [ci(out_kind), vp(self._work.ptr), ci(rows), ci(epl)]
            return head + [partial, (reduce_fn, combine_args, ((units + 7) // 8, 1, 1), (256, 1, 1), 0)]
        dsplit = plan.combine_dsplit
        combine_args = reduce_args + [ci(dsplit), vp(self._work.ptr)]
        combine_smem = min(C, 256) * 4
        combine = (reduce_fn, combine_args, (batch * Hq * dsplit, 1, 1), (256, 1, 1), combine_smem)
        return head + [partial, combine]
