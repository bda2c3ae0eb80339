"""Host-side sharding logic, including a world_size-2 gloo run on the CPU."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import pkg


def test_unit_ranges_partition_the_units():
    for n in (1, 7, 8, 16, 64, 128):
        for w in (1, 2, 3, 4, 8):
            seen = []
            for r in range(w):
                lo, hi = pkg.unit_range(n, r, w)
                seen += list(range(lo, hi))
            assert seen == list(range(n))
    assert pkg.shard_units(2, 8, 7, 8) == [(1, 6), (1, 7)]
    assert pkg.shard_units(1, 8, 3, 8) == [(0, 3)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B, Hkv = 2, 3
    units = pkg.shard_units(B, Hkv, rank, world)
    # each rank "computes" a tag for its units; the gather reassembles the whole problem in unit order
    mine = torch.tensor([b * 100 + g for b, g in units], dtype=torch.int64)
    pad = torch.full((B * Hkv,), -1, dtype=torch.int64)
    pad[: len(mine)] = mine
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad)
    t = torch.tensor([float(len(units))])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        out.put(([b[b >= 0].tolist() for b in bufs], t.item()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_shards_cover_everything():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    gathered, mx = out.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    flat = gathered[0] + gathered[1]
    assert flat == [0, 1, 2, 100, 101, 102]
    assert mx == 3.0
