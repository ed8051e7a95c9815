"""(batch, head) sharding logic with world_size 2 on CPU (gloo): ranges partition the slices, scatter/gather
round-trips, and per-rank evaluation of the oracle on a shard equals the full evaluation (no cross-slice
dependency, so no collective is needed on the data path)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from attention_autotuner_b200 import sharding


def test_slice_ranges_partition():
    for n in (1, 7, 64, 512):
        for world in (1, 2, 3, 8):
            spans = [sharding.slice_range(r, world, n) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.slice_range(2, 2, 10)
    assert sharding.heads_of(6, 10, 4).tolist() == [2, 3, 0, 1]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, L, d = 3, 3, 32, 16   # 9 slices over 2 ranks: 5 + 4
        n = B * H
        full = None
        if rank == 0:
            g = torch.Generator().manual_seed(0)
            full = torch.randn(3, n, L, d, generator=g)
        shards = [sharding.scatter_slices(full[i] if rank == 0 else None, n, (L, d), torch.float32, "cpu") for i in range(3)]
        lo, hi = sharding.slice_range(rank, world, n)
        assert shards[0].shape[0] == hi - lo
        # each rank's own slices, with the head-indexed mask rows of its range
        mask = oracle.decay_mask(H, L, L)
        heads = sharding.heads_of(lo, hi, H)
        o_shard, _ = oracle.retnet_fwd(shards[0], shards[1], shards[2], mask[heads], 0.25)
        o_full = sharding.gather_slices(o_shard, n)
        if rank == 0:
            q4 = [full[i].view(B, H, L, d) for i in range(3)]
            ref, _ = oracle.retnet_fwd(q4[0], q4[1], q4[2], mask, 0.25)
            assert torch.equal(o_full.view(B, H, L, d), ref) or torch.allclose(o_full.view(B, H, L, d), ref, atol=1e-6)
        dist.barrier()
        q.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_rank_scatter_compute_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
