"""Device side of the row-sharded pooling path. The ranks are emulated in one process on one GPU
(the kernels do not wait on one another, so this is exact): every rank's ids are routed, the two
exchanges are done by slicing, and the result is compared with the un-sharded oracle. Routing
(owner, local row, bucket order, tags) must be bit-exact against the CPU restatement."""
import numpy as np
import pytest
import torch

import orc
import pkg
from cpu_shard_ops import CpuShardOps
from test_sharded_cpu import _case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,avg", [(2, False), (8, False), (8, True), (5, False)])
def test_emulated_ranks_match_unsharded_oracle(world, avg):
    pkg.load()
    from x_deeplearning_b200 import ops, sharded
    dim, groups, per_rank = 8, 3, 5
    table, data = _case(world * 7 + int(avg), world)
    gops, cops = sharded.GpuShardOps(), CpuShardOps()
    shards = [ops.Table(torch.from_numpy(np.ascontiguousarray(table[r::world])), torch.float32) for r in range(world)]
    segments = groups * per_rank
    routed = []
    for r in range(world):
        ids, vals, off, counts = data[r]
        g = gops.route(torch.from_numpy(ids).cuda(), torch.from_numpy(vals).cuda(), torch.from_numpy(off).cuda(), world)
        c = cops.route(torch.from_numpy(ids), torch.from_numpy(vals), torch.from_numpy(off), world)
        for a, b in zip(g, c):
            assert torch.equal(a.cpu(), b), "routing differs from the CPU restatement"
        routed.append(g)
    # exchange 1 by slicing: owner w receives bucket w of every source, sources in rank order
    partial = []
    for w in range(world):
        rows, vals, tags, cnts = [], [], [], []
        for s in range(world):
            oc = routed[s][3].cpu().tolist()
            lo, hi = sum(oc[:w]), sum(oc[:w + 1])
            rows.append(routed[s][0][lo:hi]); vals.append(routed[s][1][lo:hi])
            t = routed[s][2][lo:hi]
            cnts.append(gops.tag_counts(t, segments))
        partial.append(gops.pool_partial(shards[w], torch.cat(rows), torch.cat(vals), torch.cat(cnts), dim))   # [world*segments, dim]
    # exchange 2 by slicing: source s gets its slice from every owner
    for s in range(world):
        back = torch.cat([partial[w][s * segments:(s + 1) * segments] for w in range(world)]).contiguous()
        ids, vals, off, counts = data[s]
        out = torch.zeros((per_rank, groups * dim), device="cuda")
        seg_len = torch.from_numpy(counts).cuda() if avg else None
        gops.combine(back, world, segments, dim, groups, out, seg_len, avg)
        want = np.zeros((segments, dim), np.float32)
        orc.embedding_pool(table, ids, vals, counts, [dict(udf=1 if avg else 0, out=want, col=0)])
        want = want.reshape(groups, per_rank, dim).transpose(1, 0, 2).reshape(per_rank, groups * dim)
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-5)


def test_route_large_stream_is_a_stable_partition():
    pkg.load()
    from x_deeplearning_b200 import sharded
    rng = np.random.default_rng(3)
    n, world = 300_000, 8
    counts = rng.integers(0, 40, 15000).astype(np.int32)
    counts[-1] += n - int(counts.sum()) if counts.sum() < n else 0
    n = int(counts.sum())
    ids = rng.integers(0, 1 << 40, n).astype(np.int64)
    off = np.zeros(len(counts) + 1, np.int32)
    np.cumsum(counts, out=off[1:])
    g = sharded.GpuShardOps().route(torch.from_numpy(ids).cuda(), None, torch.from_numpy(off).cuda(), world)
    c = CpuShardOps().route(torch.from_numpy(ids), None, torch.from_numpy(off), world)
    for a, b in zip(g, c):
        assert torch.equal(a.cpu(), b)
