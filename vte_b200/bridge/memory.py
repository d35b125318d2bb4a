"""Slab allocator: one large device allocation carved into aligned blocks.

Same surface as vte/bridge/memory.py:10-202 (`MemoryRegion`, `MemoryBlock`,
`SlabAllocator.initialize / allocate / free / validate_pointer / get_stats /
cleanup`): the dispatcher asks it for its scratch buffers
(`allocate(size, tag, MemoryRegion.SCRATCH)` returning an object with `.ptr`).
Blocks are aligned to 128 bytes here (the reference uses 64): bulk asynchronous
copies and 128-bit vector loads want 16, and 128 keeps every buffer on its own
L2 line.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum
from typing import Optional

from ..config import CACHE_LINE_SIZE
from .errors import CudaSafetyError


class MemoryRegion(IntEnum):
    WEIGHTS = 0
    KV_CACHE = 1
    ACTIVATIONS = 2
    SCRATCH = 3


@dataclass
class MemoryBlock:
    offset: int
    size: int
    aligned_size: int
    ptr: int
    tag: str
    region: MemoryRegion
    in_use: bool = True


class SlabAllocator:
    def __init__(self, runtime, total_vram_bytes: int, requested_pool_size: Optional[int] = None):
        self._rt = runtime
        self._total_vram = int(total_vram_bytes)
        ceiling = int(self._total_vram * 0.80)
        want = int(requested_pool_size) if requested_pool_size else int(self._total_vram * 0.85)
        self.total_size = min(want, ceiling)
        self.slab_base = 0
        self.blocks: list[MemoryBlock] = []
        self.free_list: list[tuple[int, int]] = []   # (offset, size), kept merged
        self.current_offset = 0
        self._initialized = False

    def initialize(self):
        if self._initialized:
            raise CudaSafetyError("SlabAllocator is already initialised")     # as vte/bridge/memory.py:55-56
        handle = self._rt.safe_malloc(self.total_size, "VTE_GIANT_SLAB")
        self.slab_base = handle.value if hasattr(handle, "value") else int(handle)
        self._initialized = True

    def allocate(self, size: int, tag: str, region: MemoryRegion) -> MemoryBlock:
        if not self._initialized:
            raise CudaSafetyError("SlabAllocator is not initialised")
        if size <= 0:
            raise CudaSafetyError(f"invalid allocation size {size} [{tag}]")
        need = (size + CACHE_LINE_SIZE - 1) // CACHE_LINE_SIZE * CACHE_LINE_SIZE
        # best fit among the holes left by earlier frees
        best = min((i for i, (_, sz) in enumerate(self.free_list) if sz >= need),
                   key=lambda i: self.free_list[i][1] - need, default=None)
        if best is not None:
            off, sz = self.free_list.pop(best)
            if sz > need:
                self.free_list.append((off + need, sz - need))
                self.free_list.sort()
        else:
            if self.current_offset + need > self.total_size:
                raise CudaSafetyError(f"slab exhausted: {need} bytes requested [{tag}], "
                                      f"{self.total_size - self.current_offset} left")
            off = self.current_offset
            self.current_offset += need
        block = MemoryBlock(offset=off, size=size, aligned_size=need, ptr=self.slab_base + off, tag=tag,
                            region=region)
        self._check_overlap(block)
        self.blocks.append(block)
        return block

    def _check_overlap(self, new_block: MemoryBlock):
        lo, hi = new_block.offset, new_block.offset + new_block.aligned_size
        for b in self.blocks:
            if b.in_use and lo < b.offset + b.aligned_size and b.offset < hi:
                raise CudaSafetyError(f"overlap between [{new_block.tag}] and [{b.tag}]")

    def free(self, block: MemoryBlock):
        if not block.in_use:
            raise CudaSafetyError(f"double free of [{block.tag}]")
        block.in_use = False
        self.blocks = [b for b in self.blocks if b is not block]
        self.free_list.append((block.offset, block.aligned_size))
        self._merge_adjacent_free_blocks()

    def _merge_adjacent_free_blocks(self):
        merged: list[tuple[int, int]] = []
        for off, sz in sorted(self.free_list):
            if merged and merged[-1][0] + merged[-1][1] == off:
                merged[-1] = (merged[-1][0], merged[-1][1] + sz)
            else:
                merged.append((off, sz))
        # a hole that touches the bump pointer goes back to it
        if merged and merged[-1][0] + merged[-1][1] == self.current_offset:
            self.current_offset = merged.pop()[0]
        self.free_list = merged

    def validate_pointer(self, ptr: int, size: int) -> bool:
        """True when [ptr, ptr + size) lies inside one live block."""
        if not (self.slab_base <= ptr < self.slab_base + self.total_size):
            return False
        for b in self.blocks:
            if b.in_use and b.ptr <= ptr and ptr + size <= b.ptr + b.aligned_size:
                return True
        return False

    def get_stats(self) -> dict:
        """The reference's four keys (vte/bridge/memory.py:185-193) plus the number of holes."""
        used = sum(b.aligned_size for b in self.blocks if b.in_use)
        return {"total_bytes": self.total_size, "used_bytes": used, "free_bytes": self.total_size - used,
                "active_blocks": sum(1 for b in self.blocks if b.in_use), "holes": len(self.free_list)}

    def cleanup(self):
        """Clears the bookkeeping as vte/bridge/memory.py:195-202 does and, unlike it, also hands the
        slab back: several executors share one runtime in a process here, and the runtime's own
        cleanup would otherwise be the first to free it."""
        if self._initialized and self.slab_base:
            import ctypes
            self._rt.safe_free(ctypes.c_void_p(self.slab_base), "VTE_GIANT_SLAB")
        self.blocks.clear()
        self.free_list.clear()
        self.current_offset = 0
        self.slab_base = 0
        self._initialized = False
