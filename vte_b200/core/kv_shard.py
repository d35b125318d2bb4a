"""Decode attention for one very long sequence whose KV range is split across GPUs.

Rank r of n holds positions [r * S / n, (r + 1) * S / n) of every layer's cache
(its local kv offset is S / n - 1).  Per layer each rank runs the split kernel
over its own range, reduces its splits to one unnormalised state per query head
(o[D], m, l: 6,240 bytes for 12 heads of 128), all ranks all-gather the states
with NCCL over NVLink, and every rank applies the log-sum-exp merge over the
shard axis.  No remote K/V is ever read.  The reference has no multi-GPU path;
the merge is the arithmetic of its reduce kernel
(flash_attention_split_kv_reduce.hip.template:24-66) run over shards.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from ..bridge.memory import MemoryRegion
from .decode_executor import DecodeAttentionExecutor


def kv_range_of_rank(total: int, rank: int, world: int) -> tuple[int, int]:
    """[start, end) of the positions rank `rank` owns; ranges are contiguous, cover
    0..total and differ in length by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside 0..{world - 1}")
    return rank * total // world, (rank + 1) * total // world


def sequences_of_rank(batch: int, rank: int, world: int) -> tuple[int, int]:
    """[first, last) sequence indices of rank `rank` when a batch is sharded by
    sequence (contiguous blocks, no collective)."""
    return kv_range_of_rank(batch, rank, world)


class PeerTable(ctypes.Structure):
    """Kernel argument of vteb_push_shard_state_kernel: every rank's board and flag array
    as mapped into this process (own rank: the local allocation)."""
    _fields_ = [("board", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8)]


class PairBoards(ctypes.Structure):
    """Kernel argument of vteb_split_kv_combine_push_kernel: every rank's board of tagged
    64-bit words as mapped into this process."""
    _fields_ = [("board", ctypes.c_void_p * 8)]


class KVRangeShardedDecode:
    """`exchange="nccl"`: ncclAllGather of the states.  `exchange="p2p"`: the state combine itself
    stores every value, as a 64-bit (value, step tag) word, into each rank's exported board over
    NVLink, and the merge kernel polls (bounded) the words it needs on its own board: no fence,
    no flag, one launch fewer per layer.  `exchange="p2p-flags"`: the earlier form, a push kernel
    that stores the state and then raises a flag on every peer (also the fallback of "p2p" when
    the short-list combine kernel is in use).  Both need `rendezvous` to swap the memory handles,
    at most eight ranks, one process per GPU on one node."""

    def __init__(self, hip, codegen, metadata: dict, shard_context_length: int, n_layers: int, comm, *,
                 n_kv_buffers: Optional[int] = None, num_splits: Optional[int] = None, programmatic: Optional[bool] = None,
                 exchange: str = "nccl", rendezvous=None, fused_merge: bool = True):
        self.hip, self.comm = hip, comm
        self.world = comm.world if comm is not None else (rendezvous.world if rendezvous is not None else 1)
        self.rank = comm.rank if comm is not None else (rendezvous.rank if rendezvous is not None else 0)
        if exchange not in ("nccl", "p2p", "p2p-flags"):
            raise ValueError(f"exchange must be nccl, p2p or p2p-flags, not {exchange!r}")
        if exchange != "nccl" and (rendezvous is None or self.world > 8):
            raise ValueError("the p2p exchange needs the host rendezvous and at most eight ranks")
        self.exchange, self.rdzv = exchange, rendezvous
        # "p2p" only: the combine launch also merges its slice of every rank's state (combine, exchange
        # and merge in one kernel); False leaves the merge to a launch of its own
        self.fused_merge = bool(fused_merge)
        self._peer_ptrs: list[int] = []
        self._board = None
        self.L = int(n_layers)
        self.ex = DecodeAttentionExecutor(hip, codegen, metadata, 1, shard_context_length, n_layers,
                                          n_kv_buffers=n_kv_buffers, num_splits=num_splits, emit_state=True,
                                          programmatic=programmatic, per_layer_hook=self._after_layer)
        ex = self.ex
        self.rows = ex.B * ex.Hq
        self.state_floats = self.rows * (ex.D + 2)
        A = ex.allocator.allocate
        self.gathered = A(self.L * self.world * self.state_floats * 4, "shard_states.gathered", MemoryRegion.ACTIVATIONS)
        self.merged = A(self.L * self.rows * ex.D * 4, "attention.output.merged", MemoryRegion.ACTIVATIONS)
        arch = hip.get_gpu_architecture()
        _, self._merge_fn = codegen.load_kernel_safe(hip, 'decode_attention', arch, 'vteb_merge_shard_states_kernel')
        self._stage_merged = hip.host_alloc(self.L * self.rows * ex.D * 4)
        self._stage_status = hip.host_alloc(64)          # the split kernels' status word, read back with the result
        self.tagged = False                     # the fused combine + push with tagged words is in use
        if self.exchange != "nccl" and self.world > 1:
            self._setup_peer_boards(codegen, arch)

    def _setup_peer_boards(self, codegen, arch):
        """One allocation per rank: board floats, then flags, then the step word; exported to
        the peers through the host rendezvous."""
        hip = self.hip
        self._board_floats = 2 * self.L * self.world * self.state_floats
        self._flag_ints = 2 * self.L * self.world
        board_bytes = self._board_floats * 8          # sized for 64-bit tagged words; the flag form uses half of it
        nbytes = board_bytes + self._flag_ints * 4 + 64
        self._board = hip.safe_malloc(nbytes, "shard_states.board")
        hip.safe_memset(self._board, nbytes, "shard_states.board")
        hip.synchronize()
        handles = self.rdzv.allgather(hip.ipc_export(self._board))
        table = PeerTable()
        for r in range(self.world):
            base = self._board.value if r == self.rank else hip.ipc_open(handles[r])
            if r != self.rank:
                self._peer_ptrs.append(base)
            table.board[r] = base
            table.flags[r] = base + board_bytes
        self._peers = table
        self._pair_boards = PairBoards()
        for r in range(self.world):
            self._pair_boards.board[r] = table.board[r]
        self._flags_ptr = self._board.value + board_bytes
        self._step_ptr = self._flags_ptr + self._flag_ints * 4
        _, self._push_fn = codegen.load_kernel_safe(hip, 'decode_attention', arch, 'vteb_push_shard_state_kernel')
        _, self._merge_p2p_fn = codegen.load_kernel_safe(hip, 'decode_attention', arch, 'vteb_merge_shard_states_p2p_kernel')
        _, self._advance_fn = codegen.load_kernel_safe(hip, 'decode_attention', arch, 'vteb_advance_step_kernel')
        _, self._combine_push_fn = codegen.load_kernel_safe(hip, 'decode_attention', arch, 'vteb_split_kv_combine_push_kernel')
        _, self._merge_ll_fn = codegen.load_kernel_safe(hip, 'decode_attention', arch, 'vteb_merge_shard_states_ll_kernel')
        # the fused form replaces the per-slice state combine; the short-list combine keeps the flag form
        self.tagged = self.exchange == "p2p" and self.ex.dispatcher.max_chunks > 64 and self.ex.D <= 256
        if self.tagged:
            self.ex.launch_rewriter = self._fuse_push_into_combine
        self.rdzv.barrier()          # every board is zeroed and mapped before anyone pushes

    def _after_layer(self, l: int) -> int:
        """Recorded right after layer l's split + state-combine launches: all-gather, merge."""
        ex = self.ex
        state_ptr = ex.out_all.ptr + l * ex.out_bytes
        gathered_ptr = self.gathered.ptr + l * self.world * self.state_floats * 4
        if self.world > 1 and self.exchange != "nccl":
            return self._after_layer_tagged(l) if self.tagged else self._after_layer_p2p(l, state_ptr)
        if self.world > 1:
            self.comm.all_gather_f32(state_ptr, gathered_ptr, self.state_floats)
        else:
            gathered_ptr = state_ptr               # one shard: its own state is the gathered list
        vp, ci = ctypes.c_void_p, ctypes.c_int
        args = [vp(gathered_ptr), vp(self.merged.ptr + l * self.rows * ex.D * 4), ci(self.world), ci(self.rows), ci(ex.D)]
        pdl = self.hip.programmatic_launch
        self.hip.programmatic_launch = False        # ordinary edge after a collective
        try:
            self.hip.launch_kernel_recorded(self._merge_fn, args, (self.rows, 1, 1), (ex.D, 1, 1), 0)
        finally:
            self.hip.programmatic_launch = pdl
        return 2 if self.world > 1 else 1

    def _fuse_push_into_combine(self, l: int, launches):
        """Replaces layer l's state-combine launch (pm, pl, po, state, Hq, D, C, dsplit, ticket) by the
        kernel that also stores the state into every rank's board."""
        fn, args, grid, block, smem = launches[-1]
        vp, ci = ctypes.c_void_p, ctypes.c_int
        pm, pl, po, state, hq, d, c, dsplit, ticket = args
        merged = self.merged.ptr + l * self.rows * self.ex.D * 4 if self.fused_merge else 0
        new_args = [pm, pl, po, state, self._pair_boards, hq, d, c, dsplit, ticket, ci(self.world), ci(self.rank), ci(l),
                    ci(self.L), ci(self.rows), vp(self._step_ptr), vp(self._board.value), vp(merged),
                    vp(self.ex.dispatcher.work_ptr + 4)]
        return launches[:-1] + [(self._combine_push_fn, new_args, grid, block, smem)]

    def _after_layer_tagged(self, l: int) -> int:
        ex, hip = self.ex, self.hip
        vp, ci = ctypes.c_void_p, ctypes.c_int
        if self.fused_merge:
            # the combine launch merged as well: nothing to add but the step advance
            if l == self.L - 1:
                hip.launch_kernel_recorded(self._advance_fn, [vp(self._step_ptr)], (1, 1, 1), (32, 1, 1), 0)
                return 1
            return 0
        hip.launch_kernel_recorded(self._merge_ll_fn,
                                   [vp(self._board.value), vp(self.merged.ptr + l * self.rows * ex.D * 4), ci(self.world),
                                    ci(self.rows), ci(ex.D), ci(l), ci(self.L), vp(self._step_ptr),
                                    vp(ex.dispatcher.work_ptr + 4)],
                                   (self.rows, 1, 1), (ex.D, 1, 1), 0)
        if l == self.L - 1:
            hip.launch_kernel_recorded(self._advance_fn, [vp(self._step_ptr)], (1, 1, 1), (32, 1, 1), 0)
            return 2
        return 1

    def _after_layer_p2p(self, l: int, state_ptr: int) -> int:
        ex, hip = self.ex, self.hip
        vp, ci = ctypes.c_void_p, ctypes.c_int
        pdl = hip.programmatic_launch
        hip.programmatic_launch = False
        try:
            hip.launch_kernel_recorded(self._push_fn, [vp(state_ptr), self._peers, ci(self.world), ci(self.rank), ci(l),
                                                       ci(self.L), ci(self.state_floats), vp(self._step_ptr)],
                                       (self.world, 1, 1), (256, 1, 1), 0)
            hip.launch_kernel_recorded(self._merge_p2p_fn,
                                       [vp(self._board.value), vp(self._flags_ptr), vp(self.merged.ptr + l * self.rows * ex.D * 4),
                                        ci(self.world), ci(self.rows), ci(ex.D), ci(l), ci(self.L), vp(self._step_ptr),
                                        vp(ex.dispatcher.work_ptr + 4)],
                                       (self.rows, 1, 1), (ex.D, 1, 1), 0)
            n = 2
            if l == self.L - 1:
                hip.launch_kernel_recorded(self._advance_fn, [vp(self._step_ptr)], (1, 1, 1), (32, 1, 1), 0)
                n += 1
        finally:
            hip.programmatic_launch = pdl
        return n

    def execute_decode(self, local_kv_offset: int) -> np.ndarray:
        """One decode step; returns the merged attention output [L, Hq, D] fp32
        (identical on every rank)."""
        ex = self.ex
        ex.build_decode_graph()
        ex._update_staging_buffers(np.array([local_kv_offset], dtype=np.int32))
        ex.launch_step()
        nbytes = self.L * self.rows * ex.D * 4
        self.hip.memcpy_d2h_async(self._stage_merged, ctypes.c_void_p(self.merged.ptr), nbytes, "attention output merged")
        self.hip.memcpy_d2h_async(self._stage_status, ctypes.c_void_p(ex.dispatcher.work_ptr + 4), 4, "status word output")
        self.hip.stream_synchronize()
        if ctypes.c_int.from_address(self._stage_status.value).value != 0:
            ex.dispatcher_check()                       # raises with the reason and clears the word
        flat = np.frombuffer((ctypes.c_char * nbytes).from_address(self._stage_merged.value), dtype=np.float32)
        return flat.reshape(self.L, ex.Hq, ex.D).copy()

    def launch_step(self):
        self.ex.build_decode_graph()
        self.ex.launch_step()

    def cleanup(self):
        if self._board is not None:
            self.hip.synchronize()
            self.rdzv.barrier()      # nobody is still storing into a peer's board
            for p in self._peer_ptrs:
                self.hip.ipc_close(p)
            self._peer_ptrs = []
            self.hip.safe_free(self._board, "shard_states.board")
            self._board = None
        if self._stage_merged is not None and self._stage_merged.value:
            self.hip.host_free(self._stage_merged)
            self.hip.host_free(self._stage_status)
            self._stage_merged = None
        self.ex.cleanup()
