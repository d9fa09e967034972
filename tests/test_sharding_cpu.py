"""Host-side batch sharding: plan properties, and a world_size-2 gloo run that shards a packed batch, lets each
rank transform its shard, all-gathers the padded shards and scatters them back into the original order."""
import os
import socket

import numpy as np
import pytest

from et_b200 import sharding


def test_equal_lengths_are_split_contiguously():
    shards = sharding.shard_sequences([512] * 10, 4)
    assert shards == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    assert sharding.shard_sequences([], 3) == [[], [], []]


def test_varlen_plan_covers_everything_once_and_balances():
    rng = np.random.default_rng(0)
    lens = rng.integers(32, 513, size=64).tolist()
    for world in (1, 2, 4, 8):
        shards = sharding.shard_sequences(lens, world)
        flat = sorted(i for s in shards for i in s)
        assert flat == list(range(64))
        assert all(s == sorted(s) for s in shards)
        costs = [sum(sharding.sequence_cost(lens[i]) for i in s) for s in shards]
        assert max(costs) <= 1.15 * (sum(costs) / world)
    pad, plan = sharding.gather_plan(lens, sharding.shard_sequences(lens, 4))
    assert pad == max(sum(lens[i] for i in s) for s in sharding.shard_sequences(lens, 4))
    covered = sorted((dst, n) for moves in plan for (_, dst, n) in moves)
    assert [c[0] for c in covered] == [r[0] for r in sharding.token_ranges(lens)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, lens, d, ret):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T = sum(lens)
        x = torch.arange(T * d, dtype=torch.float32).reshape(T, d)
        shards = sharding.shard_sequences(lens, world)
        ranges = sharding.token_ranges(lens)
        pad, plan = sharding.gather_plan(lens, shards)
        mine = torch.zeros((pad, d))
        off = 0
        for i in shards[rank]:
            a, b = ranges[i]
            mine[off:off + b - a] = x[a:b] * 2.0 + 1.0          # the per-shard "layer"
            off += b - a
        gathered = [torch.zeros((pad, d)) for _ in range(world)]
        dist.all_gather(gathered, mine)
        out = torch.zeros((T, d))
        for r in range(world):
            for (src, dst, n) in plan[r]:
                out[dst:dst + n] = gathered[r][src:src + n]
        ret[rank] = bool(torch.equal(out, x * 2.0 + 1.0))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_gloo_two_ranks_shard_and_gather_restores_order():
    import torch.multiprocessing as mp
    lens = [5, 33, 17, 64, 9, 40, 12]
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, lens, 8, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(100)
    assert all(p.exitcode == 0 for p in procs)
    assert ret.get(0) is True and ret.get(1) is True
