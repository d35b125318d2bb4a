"""Host-side rendezvous between the ranks of one node: a star of TCP sockets
around rank 0.  It carries the 128-byte NCCL unique id, barriers and small
gathers (timings); device data never goes through it.  The reference has no
multi-process code; this exists because one process drives one GPU here.

Environment, as set by `python -m torch.distributed.run`: RANK, WORLD_SIZE,
MASTER_ADDR, MASTER_PORT.  The listener uses a port derived from MASTER_PORT
(the launcher's own store owns MASTER_PORT itself).
"""
from __future__ import annotations

import os
import socket
import struct
import time


def _send_msg(sock: socket.socket, data: bytes) -> None:
    sock.sendall(struct.pack("!I", len(data)) + data)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("peer closed the rendezvous connection")
        buf.extend(chunk)
    return bytes(buf)


def _recv_msg(sock: socket.socket) -> bytes:
    (n,) = struct.unpack("!I", _recv_exact(sock, 4))
    return _recv_exact(sock, n)


def derived_port(master_port: int) -> int:
    return 20000 + (master_port * 7 + 4093) % 20000


class Rendezvous:
    def __init__(self, rank: int, world: int, addr: str = "127.0.0.1", port: int = 29511, timeout_s: float = 120.0):
        self.rank, self.world = int(rank), int(world)
        self.timeout_s = timeout_s
        self._peers: dict[int, socket.socket] = {}
        self._root: socket.socket | None = None
        if self.world <= 1:
            return
        if self.rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, port))
            srv.listen(self.world)
            srv.settimeout(timeout_s)
            try:
                while len(self._peers) < self.world - 1:
                    conn, _ = srv.accept()
                    conn.settimeout(timeout_s)
                    conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                    (peer_rank,) = struct.unpack("!I", _recv_exact(conn, 4))
                    self._peers[peer_rank] = conn
            finally:
                srv.close()
        else:
            deadline = time.monotonic() + timeout_s
            while True:
                try:
                    s = socket.create_connection((addr, port), timeout=5.0)
                    break
                except OSError:
                    if time.monotonic() > deadline:
                        raise TimeoutError(f"rank {rank}: rank 0 never opened {addr}:{port}")
                    time.sleep(0.05)
            s.settimeout(timeout_s)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.sendall(struct.pack("!I", self.rank))
            self._root = s

    @classmethod
    def from_env(cls, timeout_s: float = 120.0) -> "Rendezvous":
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = derived_port(int(os.environ.get("MASTER_PORT", "29500")))
        return cls(rank, world, addr, port, timeout_s)

    def allgather(self, data: bytes) -> list[bytes]:
        if self.world <= 1:
            return [data]
        if self.rank == 0:
            parts = [b""] * self.world
            parts[0] = data
            for r, s in self._peers.items():
                parts[r] = _recv_msg(s)
            blob = b"".join(struct.pack("!I", len(p)) + p for p in parts)
            for s in self._peers.values():
                _send_msg(s, blob)
            return parts
        _send_msg(self._root, data)
        blob = _recv_msg(self._root)
        parts, pos = [], 0
        for _ in range(self.world):
            (n,) = struct.unpack("!I", blob[pos:pos + 4])
            parts.append(blob[pos + 4:pos + 4 + n])
            pos += 4 + n
        return parts

    def broadcast(self, data: bytes | None) -> bytes:
        """Rank 0's bytes on every rank."""
        return self.allgather(data if self.rank == 0 and data is not None else b"")[0]

    def barrier(self) -> None:
        self.allgather(b"")

    def max_float(self, x: float) -> float:
        return max(struct.unpack("!d", p)[0] for p in self.allgather(struct.pack("!d", float(x))))

    def close(self) -> None:
        for s in list(self._peers.values()) + ([self._root] if self._root else []):
            try:
                s.close()
            except OSError:
                pass
        self._peers.clear()
        self._root = None
