"""World-size-2 gloo test of the multi-GPU partitioning (CPU ranks, oracle arithmetic): each rank computes its
head shard of a packed batch, the shards are gathered, and the result equals the unsharded computation.  No
collective is needed on the data path itself; the gather here only serves the comparison."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import kda_oracle as O
from experiment_swa_kda_b200 import sharding


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, K, V = 4, 8, 8
        cu = [0, 5, 37, 37, 70]
        d = O.make_inputs(1, 70, H, K, V, seed=3, with_state=True, n_states=4)
        b, e = sharding.head_shard(H, world, rank)
        part = {n: (t[:, b:e] if n == "h0" else t[:, :, b:e]) for n, t in d.items()}
        o, s = O.kda_recurrence_varlen(part["q"], part["k"], part["v"], part["g"], part["beta"], cu, initial_state=part["h0"])
        outs = [torch.empty_like(o) for _ in range(world)]
        sts = [torch.empty_like(s) for _ in range(world)]
        dist.all_gather(outs, o.contiguous())
        dist.all_gather(sts, s.contiguous())
        if rank == 0:
            full_o, full_s = O.kda_recurrence_varlen(d["q"], d["k"], d["v"], d["g"], d["beta"], cu, initial_state=d["h0"])
            q.put((torch.equal(torch.cat(outs, dim=2), full_o), torch.equal(torch.cat(sts, dim=1), full_s)))
    finally:
        dist.destroy_process_group()


def test_head_sharded_ranks_reproduce_the_unsharded_result():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    same_o, same_s = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same_o and same_s


def test_shard_arithmetic():
    assert [sharding.head_shard(16, 8, r) for r in range(8)] == [(2 * r, 2 * r + 2) for r in range(8)]
    assert [sharding.head_shard(3, 2, r) for r in range(2)] == [(0, 2), (2, 3)]
    with pytest.raises(ValueError):
        sharding.head_shard(3, 4, 0)
    parts = sharding.sequence_shard([8192, 300, 4000, 4100, 256], 2)
    assert sorted(sum(parts, [])) == [0, 1, 2, 3, 4]
    lens = [8192, 300, 4000, 4100, 256]
    loads = [sum(lens[i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 700
    assert [sharding.batch_shard(256, 8, r) for r in (0, 7)] == [(0, 32), (224, 256)]
