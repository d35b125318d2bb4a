"""NCCL communicator over the shim's `vteb_nccl_*` entry points.

The reference has no collective (it drives one GPU); this exists for the one
exchange step of the KV-range sharded path: an all-gather of every rank's
(o, m, l) state, a few KB per rank over NVLink.  The unique id travels through
the host rendezvous.
"""
from __future__ import annotations

import ctypes

from .errors import CudaRuntimeError, CudaSafetyError


class NcclCommunicator:
    def __init__(self, runtime, rank: int, world: int, rendezvous):
        if not (0 <= rank < world):
            raise CudaSafetyError(f"rank {rank} outside 0..{world - 1}")
        self.rt, self.rank, self.world = runtime, int(rank), int(world)
        self._lib = runtime._lib
        ident = ctypes.create_string_buffer(128)
        if rank == 0:
            self._check(self._lib.vteb_nccl_unique_id(ident), "ncclGetUniqueId")
        blob = rendezvous.broadcast(ident.raw if rank == 0 else None)
        if len(blob) != 128:
            raise CudaRuntimeError(f"NCCL unique id has {len(blob)} bytes, expected 128")
        ident = ctypes.create_string_buffer(blob, 128)
        self._comm = ctypes.c_void_p()
        self._check(self._lib.vteb_nccl_comm_init_rank(ctypes.byref(self._comm), world, ident, rank), "ncclCommInitRank")

    def _check(self, err: int, what: str):
        if err != 0:
            raise CudaRuntimeError(f"{what} returned code {err}: {self.rt._last_error()}", code=err)

    def all_gather_f32(self, send_ptr: int, recv_ptr: int, count_per_rank: int):
        """Enqueue on the runtime's stream (captured into the graph while capturing)."""
        self._check(self._lib.vteb_nccl_all_gather_f32(self._comm, ctypes.c_void_p(send_ptr), ctypes.c_void_p(recv_ptr),
                                                       count_per_rank, self.rt.stream), "ncclAllGather")

    def all_reduce_max_f32(self, send_ptr: int, recv_ptr: int, count: int):
        self._check(self._lib.vteb_nccl_all_reduce_max_f32(self._comm, ctypes.c_void_p(send_ptr), ctypes.c_void_p(recv_ptr),
                                                           count, self.rt.stream), "ncclAllReduce")

    def destroy(self):
        if self._comm:
            self._lib.vteb_nccl_comm_destroy(self._comm)
            self._comm = ctypes.c_void_p()
