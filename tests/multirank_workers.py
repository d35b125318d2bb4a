"""Child-process bodies of the multi-rank tests (CPU and GPU)."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def rendezvous_worker(rank, world, port, queue):
    from vte_b200.bridge.rendezvous import Rendezvous
    rdzv = Rendezvous(rank, world, "127.0.0.1", port, timeout_s=30)
    blob = rdzv.broadcast(b"unique-id-from-rank-0" if rank == 0 else None)
    parts = rdzv.allgather(f"rank{rank}".encode())
    rdzv.barrier()
    mx = rdzv.max_float(1.5 + rank)
    rdzv.close()
    queue.put((rank, blob, parts, mx))


def gloo_worker(rank, world, port, queue):
    """KV-range sharding and sequence sharding with the oracle's arithmetic on
    each rank and gloo as the exchange: checks the range / local-offset / merge
    logic the GPU path uses."""
    import torch
    import torch.distributed as dist
    from oracle import attention_oracle as orc
    from vte_b200.core.kv_shard import kv_range_of_rank, sequences_of_rank
    from vte_b200.workloads import DecodeConfig, make_layer_inputs

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        # --- one long sequence, KV range split over the ranks
        cfg = DecodeConfig("shard", 31, 1, 12, 2, 128, 1000, 1000, 1)
        q, k, v, off = make_layer_inputs(cfg, 0)
        total = int(off[0]) + 1
        lo, hi = kv_range_of_rank(total, rank, world)
        local_off = np.array([hi - lo - 1], dtype=np.int32)
        pm, pl, po = orc.split_kv_partial(q, k[:, lo:hi], v[:, lo:hi], local_off, cfg.scale, 4)
        # local reduce to one unnormalised state per head: [Hq, D + 2] = o, m, l
        M = pm.max(axis=2)
        w = np.exp(pm - M[..., None])
        state = np.concatenate([(po * w[..., None]).sum(axis=2), M[..., None], (pl * w).sum(axis=2)[..., None]], axis=-1)[0]
        mine = torch.from_numpy(np.ascontiguousarray(state, dtype=np.float32))
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        states = [(g[:, 128].numpy(), g[:, 129].numpy(), g[:, :128].numpy()) for g in gathered]
        merged = orc.merge_shard_states(states)
        ref = orc.decode_attention(q, k, v, off)[0]
        err_kv = float(np.abs(merged - ref).max())

        # --- a ragged batch sharded by sequence: no exchange needed for the result itself
        cfg2 = DecodeConfig("seqshard", 32, 6, 8, 2, 64, 5, 200, 1)
        q2, k2, v2, off2 = make_layer_inputs(cfg2, 0)
        a, b = sequences_of_rank(cfg2.batch, rank, world)
        out_local = orc.decode_attention(q2[a:b], k2[a:b], v2[a:b], off2[a:b])
        t = torch.from_numpy(out_local)
        parts = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        full = np.concatenate([p.numpy() for p in parts], axis=0)
        err_seq = float(np.abs(full - orc.decode_attention(q2, k2, v2, off2)).max())
        queue.put((rank, err_kv, err_seq))
    finally:
        dist.destroy_process_group()


def gpu_kv_shard_main():
    """One rank of the KV-range sharded GPU path (RANK / WORLD_SIZE / LOCAL_RANK /
    MASTER_ADDR / MASTER_PORT in the environment)."""
    from oracle import attention_oracle as orc
    from vte_b200.bridge import CudaRuntime
    from vte_b200.bridge.nccl import NcclCommunicator
    from vte_b200.bridge.rendezvous import Rendezvous
    from vte_b200.compiler import CodegenEngine
    from vte_b200.core.kv_shard import KVRangeShardedDecode, kv_range_of_rank
    from vte_b200.workloads import DecodeConfig, make_layer_inputs

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    total = int(os.environ.get("VTEB_TEST_CONTEXT", "16384"))
    rdzv = Rendezvous.from_env(timeout_s=120)
    rt = CudaRuntime(device_index=int(os.environ.get("LOCAL_RANK", rank)))
    rt.initialize()
    exchange = os.environ.get("VTEB_TEST_EXCHANGE", "nccl")
    comm = NcclCommunicator(rt, rank, world, rdzv) if exchange == "nccl" else None
    cfg = DecodeConfig("c5_small", 5, 1, 12, 2, 128, total, total, 2)
    meta = {'attention.head_count': 12, 'attention.head_count_kv': 2, 'attention.key_length': 128}
    lo, hi = kv_range_of_rank(total, rank, world)
    sh = KVRangeShardedDecode(rt, CodegenEngine(), meta, hi - lo, cfg.layers, comm, num_splits=int(os.environ.get("VTEB_TEST_SPLITS", "16")), exchange=exchange,
                              rendezvous=rdzv, fused_merge=os.environ.get("VTEB_TEST_FUSED_MERGE", "1") == "1")
    if exchange == "p2p" and os.environ.get("VTEB_TEST_EXPECT_TAGGED") == "1":
        assert sh.tagged, "expected the fused combine + push"
    refs = []
    for l in range(cfg.layers):
        q, k, v, off = make_layer_inputs(cfg, l)
        shard_k = np.zeros((1, hi - lo, 2, 128), np.float16); shard_k[0] = k[0, lo:hi]
        shard_v = np.zeros((1, hi - lo, 2, 128), np.float16); shard_v[0] = v[0, lo:hi]
        sh.ex.upload_layer(l, q, shard_k, shard_v)
        refs.append(orc.decode_attention(q, k, v, off)[0])
    worst = 0.0
    for _ in range(4):                                   # replays: both board parities, same result every time
        out = sh.execute_decode(hi - lo - 1)
        for l in range(cfg.layers):
            max_abs, rel = orc.parity_metrics(out[l][None], refs[l][None])
            worst = max(worst, max_abs)
            assert max_abs <= 2e-3 and rel <= 1e-2, (rank, l, max_abs, rel)
    rdzv.barrier()
    sh.cleanup()
    if comm is not None:
        comm.destroy()
    rt.cleanup()
    rdzv.close()
    print(f"rank {rank}/{world} ok max_abs={worst:.3e}", flush=True)


if __name__ == "__main__":
    gpu_kv_shard_main()
