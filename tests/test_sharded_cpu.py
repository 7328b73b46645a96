"""The exchange logic of the row-sharded pooling path with 2 gloo ranks on the CPU: the pooled
vectors must equal the un-sharded oracle, and ids must reach exactly the owner the rule names."""
import os
import socket
import sys

import numpy as np
import torch
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _case(seed, world, rows_total=4000, dim=8, groups=3, per_rank=5):
    rng = np.random.default_rng(seed)
    table = rng.normal(0, 0.5, (rows_total, dim)).astype(np.float32)
    data = []
    for r in range(world):
        counts = rng.integers(0, 6, groups * per_rank).astype(np.int32)       # group-major segments, some empty
        n = int(counts.sum())
        ids = rng.integers(0, rows_total, n).astype(np.int64)
        vals = rng.normal(1, 0.3, n).astype(np.float32)
        off = np.zeros(len(counts) + 1, np.int32)
        np.cumsum(counts, out=off[1:])
        data.append((ids, vals, off, counts))
    return table, data


def _worker(rank, world, port, seed, avg, ret):
    sys.path.insert(0, HERE)
    import torch.distributed as dist
    import pkg
    pkg.load()
    from x_deeplearning_b200 import sharded
    import orc
    from cpu_shard_ops import CpuShardOps
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    table, data = _case(seed, world)
    dim, groups, per_rank = table.shape[1], 3, 5
    shard = np.ascontiguousarray(table[rank::world])                        # row r lives on rank r % world at r // world
    ids, vals, off, counts = data[rank]
    out = torch.zeros((per_rank, groups * dim), dtype=torch.float32)
    stats = sharded.sharded_pool(sharded.DistComm(), CpuShardOps(), shard, dim, torch.from_numpy(ids), torch.from_numpy(vals),
                                 torch.from_numpy(off), groups, out, avg=avg)
    want = np.zeros((groups * per_rank, dim), np.float32)
    orc.embedding_pool(table, ids, vals, counts, [dict(udf=1 if avg else 0, out=want, col=0)])
    want = want.reshape(groups, per_rank, dim).transpose(1, 0, 2).reshape(per_rank, groups * dim)
    err = float(np.abs(out.numpy() - want).max())
    ret[rank] = (err, stats["routed_bytes"])
    dist.destroy_process_group()


def _worker_tables(rank, world, port, seed, with_values, ret):
    """Two tables of different sizes and group counts through one routing pass and one pair of exchanges."""
    sys.path.insert(0, HERE)
    import torch.distributed as dist
    import pkg
    pkg.load()
    from x_deeplearning_b200 import sharded
    import orc
    from cpu_shard_ops import CpuShardOps
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    dim, per_rank = 8, 5
    cases = [_case(seed, world, rows_total=4000, groups=3), _case(seed + 50, world, rows_total=777, groups=2)]
    groups = [3, 2]
    shards = [np.ascontiguousarray(table[rank::world]) for table, _ in cases]
    mine = [data[rank] for _, data in cases]
    out = torch.zeros((per_rank, sum(groups) * dim), dtype=torch.float32)
    stats = sharded.sharded_pool_tables(
        sharded.DistComm(), CpuShardOps(), shards, dim, [torch.from_numpy(m[0]) for m in mine],
        [torch.from_numpy(m[1]) if with_values else None for m in mine], [torch.from_numpy(m[2]) for m in mine], groups, out)
    want = []
    for (table, _), (ids, vals, off, counts), g in zip(cases, mine, groups):
        w = np.zeros((g * per_rank, dim), np.float32)
        orc.embedding_pool(table, ids, vals if with_values else np.ones(len(ids), np.float32), counts, [dict(udf=0, out=w, col=0)])
        want.append(w.reshape(g, per_rank, dim).transpose(1, 0, 2).reshape(per_rank, g * dim))
    err = float(np.abs(out.numpy() - np.concatenate(want, axis=1)).max())
    ret[rank] = (err, stats["routed_bytes"])
    dist.destroy_process_group()


def _run(world, seed, avg):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, seed, avg, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        # partial sums are added owner by owner: equal to the sequential sum up to fp32 re-association
        assert ret[r][0] <= 1e-5, ret[r]


def test_two_ranks_sum():
    _run(2, 0, False)


def test_two_ranks_avg():
    _run(2, 1, True)


def test_three_ranks_sum():
    _run(3, 2, False)


def _run_tables(world, seed, with_values):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker_tables, args=(world, port, seed, with_values, ret), nprocs=world, join=True)
    got = dict(ret)
    assert len(got) == world
    for r in range(world):
        assert got[r][0] <= 1e-5, got[r]
    return got


def test_two_tables_one_exchange():
    _run_tables(2, 5, True)


def test_two_tables_without_values_route_fewer_bytes():
    a = _run_tables(2, 6, False)
    b = _run_tables(2, 6, True)
    for r in range(2):
        assert a[r][1] * 12 == b[r][1] * 8             # 8 bytes per routed id instead of 12


def test_routing_rule_is_bit_exact():
    sys.path.insert(0, HERE)
    import orc
    ids = np.array([0, 1, 7, 8, 9, (1 << 40) + 3, -1], np.int64)
    owner, local = orc.route(ids, 8)
    u = ids.astype(np.uint64)
    np.testing.assert_array_equal(owner, (u % np.uint64(8)).astype(np.int32))
    np.testing.assert_array_equal(local, (u // np.uint64(8)).astype(np.int64))
