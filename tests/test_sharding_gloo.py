"""World-size-2 check of the sharding helpers on CPU (gloo): the shards cover the
batch exactly once and the cross-rank reductions agree with a single process."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from natten_mps_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)                      # every rank seeds the full tensors
    q, k, v = [rng.standard_normal((5, 12, 2, 8)) for _ in range(3)]
    sl = sharding.batch_slice(5, rank, world)
    out, _ = oracle.na_forward(q[sl], k[sl], v[sl], kernel_size=5)
    total = sharding.reduce_sum([float(out.sum()), float(sl.stop - sl.start)])
    slowest = sharding.reduce_max([float(rank + 1)])
    if rank == 0:
        ret["sum"], ret["count"], ret["max"] = total[0], total[1], slowest[0]
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shards_cover_the_batch():
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        rng = np.random.default_rng(0)
        q, k, v = [rng.standard_normal((5, 12, 2, 8)) for _ in range(3)]
        full, _ = oracle.na_forward(q, k, v, kernel_size=5)
        assert ret["count"] == 5
        assert abs(ret["sum"] - float(full.sum())) < 1e-9
        assert ret["max"] == 2.0


def test_assign_units_balances_ragged_lengths():
    lens = [16384, 4096, 9000, 12000, 5000, 15000, 7000, 8000]
    owned = sharding.assign_units(lens, 4)
    assert sorted(i for u in owned for i in u) == list(range(8))
    loads = [sum(lens[i] for i in u) for u in owned]
    assert max(loads) - min(loads) <= max(lens)
    assert sharding.assign_units([1, 1, 1, 1], 2) == [[0, 2], [1, 3]]
    assert [sharding.batch_slice(5, r, 2) for r in range(2)] == [slice(0, 3), slice(3, 5)]
