"""world_size-2 tests on CPU: the host rendezvous, and the sharding / merge logic
of the two multi-GPU modes with gloo as the exchange."""
import multiprocessing as mp
import socket

import pytest

from tests import multirank_workers as workers
from vte_b200.core.kv_shard import kv_range_of_rank, sequences_of_rank


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(target, world=2, timeout=180):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=timeout) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    return sorted(results)


def test_rendezvous_two_ranks():
    res = _run(workers.rendezvous_worker)
    for rank, blob, parts, mx in res:
        assert blob == b"unique-id-from-rank-0"
        assert parts == [b"rank0", b"rank1"]
        assert mx == 2.5


def test_gloo_kv_range_and_sequence_sharding():
    res = _run(workers.gloo_worker)
    for rank, err_kv, err_seq in res:
        assert err_kv < 1e-5, (rank, err_kv)
        assert err_seq == 0.0, (rank, err_seq)


def test_shard_ranges_partition_exactly():
    for total in (1, 7, 64, 1000, 1048576):
        for world in (1, 2, 3, 4, 8):
            spans = [kv_range_of_rank(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert sequences_of_rank(64, 3, 8) == (24, 32)
    with pytest.raises(ValueError):
        kv_range_of_rank(10, 2, 2)


def test_bench_sharding_helpers():
    """Pieces of bench.py's sharded block that need no GPU: the longest-first deal of sequences to
    ranks, and the guard that turns one rank's failure into the same error record on every rank."""
    import importlib.util
    import numpy as np
    from pathlib import Path
    spec = importlib.util.spec_from_file_location("bench_module", Path(__file__).resolve().parent.parent / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from vte_b200.bridge.rendezvous import Rendezvous
    from vte_b200.workloads import CONFIGS, draw_context_lengths

    lengths = draw_context_lengths(CONFIGS["c3"])
    for world in (2, 4, 8):
        parts = bench.balanced_assignment(lengths, world)
        assert sorted(int(b) for p in parts for b in p) == list(range(64))          # every sequence exactly once
        assert all(len(p) == 64 // world for p in parts)
        loads = [int(lengths[p].astype(np.int64).sum()) for p in parts]
        assert max(loads) / (sum(loads) / world) < 1.03                              # contiguous blocks: up to 1.27
    rdzv = Rendezvous(0, 1)
    assert bench.guarded(rdzv, lambda: {"value": 1.0}) == {"value": 1.0}

    def boom():
        raise RuntimeError("no device")
    rec = bench.guarded(rdzv, boom)
    assert "error" in rec and "no device" in rec["error"]
