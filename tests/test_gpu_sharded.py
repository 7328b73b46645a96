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


class _SelfComm:
    """A world of one rank: both exchanges hand the buffers back."""
    world, rank = 1, 0

    def exchange_counts(self, counts):
        return counts.clone()

    def all_to_all_v(self, send, send_counts, recv_counts):
        return send.clone()

    def all_to_all_equal(self, send):
        return send.clone()


@pytest.mark.parametrize("with_values", [True, False])
def test_several_tables_through_one_routing_pass(with_values):
    pkg.load()
    from x_deeplearning_b200 import ops, sharded
    dim, per_rank, groups = 8, 5, [3, 2, 4]
    cases = [_case(11 + t, 1, rows_total=r, groups=g) for t, (r, g) in enumerate(zip([4000, 777, 50], groups))]
    tables = [ops.Table(torch.from_numpy(table), torch.float32) for table, _ in cases]
    mine = [data[0] for _, data in cases]
    out = torch.zeros((per_rank, sum(groups) * dim), device="cuda")
    sharded.sharded_pool_tables(_SelfComm(), sharded.GpuShardOps(), tables, dim, [torch.from_numpy(m[0]).cuda() for m in mine],
                                [torch.from_numpy(m[1]).cuda() if with_values else None for m in mine],
                                [torch.from_numpy(m[2]).cuda() for m in mine], groups, out)
    want = []
    for (table, _), (ids, vals, off, counts), g in zip(cases, mine, groups):
        w = np.zeros((g * per_rank, dim), np.float32)
        orc.embedding_pool(table, ids, vals if with_values else np.ones(len(ids), np.float32), counts, [dict(udf=0, out=w, col=0)])
        want.append(w.reshape(g, per_rank, dim).transpose(1, 0, 2).reshape(per_rank, g * dim))
    np.testing.assert_allclose(out.cpu().numpy(), np.concatenate(want, axis=1), rtol=1e-5, atol=1e-5)


def test_owner_side_pooling_of_several_sources_and_tables_matches_the_cpu_restatement():
    pkg.load()
    from x_deeplearning_b200 import ops, sharded
    rng = np.random.default_rng(5)
    dim, sources, table_segments = 8, 3, [6, 4]
    S = sum(table_segments)
    shards_np = [rng.normal(0, 0.5, (300, dim)).astype(np.float32), rng.normal(0, 0.5, (40, dim)).astype(np.float32)]
    counts = rng.integers(0, 5, sources * S).astype(np.int32)
    off = np.zeros(len(counts) + 1, np.int32)
    np.cumsum(counts, out=off[1:])
    rows = np.zeros(int(off[-1]), np.int64)
    for s in range(sources):
        lo = s * S
        for shard, n in zip(shards_np, table_segments):
            a, b = off[lo], off[lo + n]
            rows[a:b] = rng.integers(0, len(shard), b - a)
            lo += n
    vals = rng.normal(1, 0.3, len(rows)).astype(np.float32)
    want = CpuShardOps().pool_partial_tables(shards_np, torch.from_numpy(rows), torch.from_numpy(vals), torch.from_numpy(off),
                                             sources, table_segments, dim)
    tables = [ops.Table(torch.from_numpy(t), torch.float32) for t in shards_np]
    got = sharded.GpuShardOps().pool_partial_tables(tables, torch.from_numpy(rows).cuda(), torch.from_numpy(vals).cuda(),
                                                    torch.from_numpy(off).cuda(), sources, table_segments, dim)
    np.testing.assert_allclose(got.cpu().numpy(), want.numpy(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("world,dim,out_dtype,avg", [(8, 32, torch.float16, False), (3, 8, torch.float32, True),
                                                     (2, 6, torch.float32, False), (4, 12, torch.float16, True)])
def test_combine_matches_the_cpu_restatement(world, dim, out_dtype, avg):
    """Owner-ordered sum of the returned partial vectors: the 16-byte path (dim % 4 == 0) and the element path."""
    pkg.load()
    from x_deeplearning_b200 import sharded
    rng = np.random.default_rng(world * 100 + dim)
    groups, rows = 5, 37
    segments = groups * rows
    partial = rng.normal(0, 1, (world * segments, dim)).astype(np.float32)
    seg_len = rng.integers(0, 9, segments).astype(np.int32)
    want = torch.zeros((rows, groups * dim), dtype=torch.float32)
    CpuShardOps().combine(torch.from_numpy(partial), world, segments, dim, groups, want, torch.from_numpy(seg_len), avg)
    out = torch.zeros((rows, groups * dim), dtype=out_dtype, device="cuda")
    sharded.GpuShardOps().combine(torch.from_numpy(partial).cuda(), world, segments, dim, groups, out,
                                  torch.from_numpy(seg_len).cuda() if avg else None, avg)
    if out_dtype == torch.float32:
        assert torch.equal(out.cpu(), want)                      # same adds in the same order
    else:
        assert torch.equal(out.cpu(), want.to(torch.float16))


@pytest.mark.parametrize("world", [8, 5])
def test_packed_records_carry_the_same_routing(world):
    """(segment << 32) | local row per id: the same buckets as rows and tags apart, bit for bit, with and
    without per-id values; a local row beyond 31 bits travels as 0x7fffffff (a row no shard holds)."""
    pkg.load()
    from x_deeplearning_b200 import sharded
    rng = np.random.default_rng(30 + world)
    counts = rng.integers(0, 40, 9000).astype(np.int32)
    n = int(counts.sum())
    ids = rng.integers(0, 1 << 33, n).astype(np.int64)
    ids[:5] = [(1 << 50) + 3, -1, 0, (1 << 31) * world - 1, (1 << 31) * world]
    vals = rng.normal(1, 0.3, n).astype(np.float32)
    off = np.zeros(len(counts) + 1, np.int32)
    np.cumsum(counts, out=off[1:])
    gops, cops = sharded.GpuShardOps(), CpuShardOps()
    for v in (vals, None):
        g = gops.route_packed(torch.from_numpy(ids).cuda(), None if v is None else torch.from_numpy(v).cuda(),
                              torch.from_numpy(off).cuda(), world)
        c = cops.route_packed(torch.from_numpy(ids), None if v is None else torch.from_numpy(v), torch.from_numpy(off), world)
        assert torch.equal(g[0].cpu(), c[0]) and torch.equal(g[2].cpu(), c[2])
        assert (g[1] is None and c[1] is None) or torch.equal(g[1].cpu(), c[1])
        rows, tags = gops.unpack(g[0])
        crows, ctags = cops.unpack(c[0])
        assert torch.equal(rows.cpu(), crows) and torch.equal(tags.cpu(), ctags)
        # against the unpacked routing
        r = gops.route(torch.from_numpy(ids).cuda(), None, torch.from_numpy(off).cuda(), world)
        assert torch.equal(tags, r[2])
        big = r[0].cpu().numpy().astype(np.uint64) >= np.uint64(0x7fffffff)
        assert np.array_equal(rows.cpu().numpy()[~big], r[0].cpu().numpy()[~big].astype(np.int32))
        assert (rows.cpu().numpy()[big] == 0x7fffffff).all() and big.sum() >= 2


def test_segment_lengths_of_all_sources_in_one_launch():
    pkg.load()
    from x_deeplearning_b200 import sharded
    rng = np.random.default_rng(77)
    segments, source_counts = 500, [1200, 0, 37, 4000, 1]
    tags = np.concatenate([np.sort(rng.integers(0, segments, n)) for n in source_counts]).astype(np.int32)
    got = sharded.GpuShardOps().tag_counts_sources(torch.from_numpy(tags).cuda(), source_counts, segments)
    want = CpuShardOps().tag_counts_sources(torch.from_numpy(tags), source_counts, segments)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("world,dim,out_dtype,avg", [(8, 32, torch.float16, False), (3, 8, torch.float32, True),
                                                     (5, 12, torch.float16, False)])
def test_combine_of_fp16_partials_accumulates_in_fp32_in_owner_order(world, dim, out_dtype, avg):
    """Partials that crossed the wire as fp16: the 16-byte path (dim % 8 == 0) and the element path."""
    pkg.load()
    from x_deeplearning_b200 import sharded
    rng = np.random.default_rng(world * 10 + dim)
    groups, rows = 5, 41
    segments = groups * rows
    partial = rng.normal(0, 1, (world * segments, dim)).astype(np.float16)
    seg_len = rng.integers(0, 9, segments).astype(np.int32)
    want = torch.zeros((rows, groups * dim), dtype=torch.float32)
    CpuShardOps().combine(torch.from_numpy(partial.astype(np.float32)), world, segments, dim, groups, want,
                          torch.from_numpy(seg_len), avg)
    out = torch.zeros((rows, groups * dim), dtype=out_dtype, device="cuda")
    sharded.GpuShardOps(partial_dtype="f16").combine(torch.from_numpy(partial).cuda(), world, segments, dim, groups, out,
                                                     torch.from_numpy(seg_len).cuda() if avg else None, avg)
    assert torch.equal(out.cpu(), want.to(out_dtype))


def test_tags_from_a_peer_outside_the_segment_range_are_ignored():
    pkg.load()
    from x_deeplearning_b200 import sharded
    segments, source_counts = 50, [6, 5]
    tags = np.array([0, 3, 3, 50, -1, 49, 7, 1 << 30, 7, 7, 0], np.int32)
    got = sharded.GpuShardOps().tag_counts_sources(torch.from_numpy(tags).cuda(), source_counts, segments).cpu().numpy()
    want = np.zeros(2 * segments, np.int32)
    for s, (lo, hi) in enumerate([(0, 6), (6, 11)]):
        for t in tags[lo:hi]:
            if 0 <= t < segments:
                want[s * segments + t] += 1
    np.testing.assert_array_equal(got, want)
    one = sharded.GpuShardOps().tag_counts(torch.from_numpy(tags).cuda(), segments).cpu().numpy()
    np.testing.assert_array_equal(one, want[:segments] + want[segments:])


@pytest.mark.parametrize("partial_dtype", ["f16", "f32"])
def test_large_table_configuration_shape_on_one_rank(partial_dtype):
    """The large-table configuration's shape on a world of one rank: dim 32 fp16 tables, 4096 samples x 40 feature
    groups over 4 tables, Zipf(1.05) ids, id lists of 1..30, through the whole path (route, unpack, counts, owner
    pooling, combine) against the un-sharded oracle."""
    pkg.load()
    from x_deeplearning_b200 import ops, sharded, workloads
    rng = np.random.default_rng(42)
    n_tables, gpt, dim, B, rows_total = 4, 10, 32, 4096, 300_000
    tables_np = [workloads.fp16_round(rng.normal(0, 0.01, (rows_total, dim))) for _ in range(n_tables)]
    tables = [ops.Table(torch.from_numpy(t), torch.float16) for t in tables_np]
    feeds = []
    for t in range(n_tables):
        counts = rng.integers(1, 31, gpt * B).astype(np.int32)
        ids = workloads.zipf_ids(rng, rows_total, int(counts.sum()), 1.05)
        off = np.zeros(len(counts) + 1, np.int32)
        np.cumsum(counts, out=off[1:])
        feeds.append((ids, counts, off))
    out = torch.zeros((B, n_tables * gpt * dim), dtype=torch.float16, device="cuda")
    sharded.sharded_pool_tables(_SelfComm(), sharded.GpuShardOps(partial_dtype=partial_dtype), tables, dim,
                                [torch.from_numpy(f[0]).cuda() for f in feeds], [None] * n_tables,
                                [torch.from_numpy(f[2]).cuda() for f in feeds], [gpt] * n_tables, out)
    got = out.float().cpu().numpy()
    for t, (ids, counts, off) in enumerate(feeds):
        want = np.zeros((gpt * B, dim), np.float32)
        mag = np.zeros((gpt * B, dim), np.float32)
        ones = np.ones(len(ids), np.float32)
        orc.embedding_pool(tables_np[t], ids, ones, counts, [dict(udf=0, out=want, col=0)])
        orc.embedding_pool(np.abs(tables_np[t]), ids, ones, counts, [dict(udf=0, out=mag, col=0)])
        want = want.reshape(gpt, B, dim).transpose(1, 0, 2).reshape(B, gpt * dim)
        mag = mag.reshape(gpt, B, dim).transpose(1, 0, 2).reshape(B, gpt * dim)
        err = np.abs(got[:, t * gpt * dim:(t + 1) * gpt * dim] - want)
        # one fp16 rounding of the result (and one of the partial sum when it travels as fp16)
        tol = (2.0 if partial_dtype == "f16" else 1.0) * 2.0 ** -11
        assert (err <= tol * np.maximum(mag, 1e-6)).all(), float((err / np.maximum(mag, 1e-6)).max())


@pytest.mark.parametrize("partial_dtype", ["f16", "f32"])
def test_one_call_sharded_step_on_one_rank_matches_the_unsharded_oracle(partial_dtype):
    """xb_sharded_pool (context owned by the library, fixed-capacity buckets, no host synchronisation) on a world of
    one rank at the large-table configuration's shape, twice in a row with different ids (the context's buffers
    keep the previous step's contents)."""
    pkg.load()
    from x_deeplearning_b200 import ops, sharded, workloads
    rng = np.random.default_rng(43)
    n_tables, gpt, dim, B, rows_total = 4, 10, 32, 2048, 200_000
    tables_np = [workloads.fp16_round(rng.normal(0, 0.01, (rows_total, dim))) for _ in range(n_tables)]
    tables = [ops.Table(torch.from_numpy(t), torch.float16) for t in tables_np]
    ctx = sharded.ShardContext(0, 1, tables, [gpt * B] * n_tables, dim, max_ids=n_tables * gpt * B * 30,
                               partial_dtype=partial_dtype)
    assert ctx.bucket_capacity >= n_tables * gpt * B * 30 + 1
    out = torch.zeros((B, n_tables * gpt * dim), dtype=torch.float16, device="cuda")
    for step in range(2):
        feeds = []
        for t in range(n_tables):
            counts = rng.integers(0 if step else 1, 31, gpt * B).astype(np.int32)       # second step: some empty segments
            ids = workloads.zipf_ids(rng, rows_total, int(counts.sum()), 1.05)
            feeds.append((ids, counts))
        all_ids = np.concatenate([f[0] for f in feeds])
        all_counts = np.concatenate([f[1] for f in feeds])
        off = np.zeros(len(all_counts) + 1, np.int32)
        np.cumsum(all_counts, out=off[1:])
        if step == 1:
            ctx.profile(True)                       # phase timing changes nothing but the event records
        ctx.pool(torch.from_numpy(all_ids).cuda(), torch.from_numpy(off).cuda(), n_tables * gpt, out)
        torch.cuda.synchronize()
        assert not ctx.overflow()
        if step == 1:
            phases = ctx.phase_ms()
            assert list(phases) == list(ctx.PHASES) and all(v >= 0.0 for v in phases.values()) and sum(phases.values()) > 0.0
            ctx.profile(False)
        got = out.float().cpu().numpy()
        for t, (ids, counts) in enumerate(feeds):
            want = np.zeros((gpt * B, dim), np.float32)
            mag = np.zeros((gpt * B, dim), np.float32)
            ones = np.ones(len(ids), np.float32)
            orc.embedding_pool(tables_np[t], ids, ones, counts, [dict(udf=0, out=want, col=0)])
            orc.embedding_pool(np.abs(tables_np[t]), ids, ones, counts, [dict(udf=0, out=mag, col=0)])
            want = want.reshape(gpt, B, dim).transpose(1, 0, 2).reshape(B, gpt * dim)
            mag = mag.reshape(gpt, B, dim).transpose(1, 0, 2).reshape(B, gpt * dim)
            err = np.abs(got[:, t * gpt * dim:(t + 1) * gpt * dim] - want)
            tol = (2.0 if partial_dtype == "f16" else 1.0) * 2.0 ** -11
            assert (err <= tol * np.maximum(mag, 1e-6)).all(), float((err / np.maximum(mag, 1e-6)).max())
    ctx.close()


def test_two_steps_in_flight_give_the_same_bits_as_one_at_a_time():
    """xb_sharded_pool_begin / _finish: begin(i+1) on a side stream before finish(i) on the main stream, different ids
    every step; the results equal those of the one-call step bit for bit, and a third begin is refused."""
    pkg.load()
    from x_deeplearning_b200 import capi, ops, sharded, workloads
    rng = np.random.default_rng(47)
    n_tables, gpt, dim, B, rows_total = 2, 6, 32, 1024, 50_000
    tables = [ops.Table(torch.from_numpy(workloads.fp16_round(rng.normal(0, 0.01, (rows_total, dim)))), torch.float16)
              for _ in range(n_tables)]
    ctx = sharded.ShardContext(0, 1, tables, [gpt * B] * n_tables, dim, max_ids=n_tables * gpt * B * 20)
    steps = []
    for _ in range(5):
        counts = rng.integers(0, 21, n_tables * gpt * B).astype(np.int32)
        ids = workloads.zipf_ids(rng, rows_total, int(counts.sum()), 1.05)
        off = np.zeros(len(counts) + 1, np.int32)
        np.cumsum(counts, out=off[1:])
        steps.append((torch.from_numpy(ids).cuda(), torch.from_numpy(off).cuda()))
    G = n_tables * gpt
    want = []
    for ids, off in steps:
        out = torch.zeros((B, G * dim), dtype=torch.float16, device="cuda")
        ctx.pool(ids, off, G, out)
        want.append(out)
    torch.cuda.synchronize()
    side, main = torch.cuda.Stream(), torch.cuda.current_stream()
    side.wait_stream(main)
    got = [torch.zeros((B, G * dim), dtype=torch.float16, device="cuda") for _ in steps]
    with torch.cuda.stream(side):
        ctx.begin(*steps[0])
    for i in range(len(steps)):
        if i + 1 < len(steps):
            with torch.cuda.stream(side):
                ctx.begin(*steps[i + 1])
                if i == 0:
                    with pytest.raises(capi.XbError, match="already in flight"):
                        ctx.begin(*steps[2])
        ctx.finish(G, got[i])
    main.wait_stream(side)
    torch.cuda.synchronize()
    assert not ctx.overflow() and ops.device_status() == 0
    for w, g in zip(want, got):
        assert torch.equal(w, g)
    with pytest.raises(capi.XbError, match="no step has been begun"):
        ctx.finish(G, got[0])
    # three stages on three streams: begin(i+2), pool(i+1), combine(i)
    s_pool = torch.cuda.Stream()
    side.wait_stream(main); s_pool.wait_stream(main)
    got3 = [torch.zeros((B, G * dim), dtype=torch.float16, device="cuda") for _ in steps]
    n = len(steps)

    def begin(i):
        with torch.cuda.stream(side):
            ctx.begin(*steps[i])

    def pool():
        with torch.cuda.stream(s_pool):
            ctx.pool_stage()
    begin(0); begin(1); pool()
    for i in range(n):
        if i + 2 < n:
            begin(i + 2)
        if i + 1 < n:
            pool()
        ctx.combine(G, got3[i])
    main.wait_stream(side); main.wait_stream(s_pool)
    torch.cuda.synchronize()
    assert not ctx.overflow() and ops.device_status() == 0
    for w, g in zip(want, got3):
        assert torch.equal(w, g)
    with pytest.raises(capi.XbError, match="no pooled step is waiting"):
        ctx.combine(G, got3[0])
    ctx.close()


def test_fixed_capacity_buckets_carry_the_same_records_and_flag_overflow():
    """xb_route_ids_padded against the compact packed routing: same records in the same order behind each bucket's
    count; a capacity that is too small cuts the bucket and raises the flag."""
    pkg.load()
    from x_deeplearning_b200 import capi, ops, sharded
    L = capi.lib()
    rng = np.random.default_rng(9)
    world = 4
    counts = rng.integers(0, 30, 3000).astype(np.int32)
    n = int(counts.sum())
    ids = rng.integers(0, 1 << 33, n).astype(np.int64)
    ids[: n // 3] = (ids[: n // 3] // world) * world + 1            # owner 1 is hot
    off = np.zeros(len(counts) + 1, np.int32)
    np.cumsum(counts, out=off[1:])
    d_ids, d_off = torch.from_numpy(ids).cuda(), torch.from_numpy(off).cuda()
    compact, _, owner_counts = sharded.GpuShardOps().route_packed(d_ids, None, d_off, world)
    oc = owner_counts.cpu().numpy()
    need = int(L.xb_route_scratch_bytes(n, world))
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    for cap, expect_overflow in ((int(oc.max()) + 1, False), (int(oc.max()) - 5, True)):
        rec = torch.full((world * cap,), -7, dtype=torch.int64, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        capi.check(L.xb_route_ids_padded(ops.ptr(d_ids), ops.ptr(d_off), len(counts), n, world, cap, ops.ptr(rec),
                                         ops.ptr(flag), ops.ptr(scratch), need, ops.stream()))
        torch.cuda.synchronize()
        assert bool(flag.item()) == expect_overflow
        r, c = rec.cpu().numpy().reshape(world, cap), compact.cpu().numpy()
        pos = 0
        for w in range(world):
            kept = min(int(oc[w]), cap - 1)
            assert r[w, 0] == kept
            np.testing.assert_array_equal(r[w, 1:1 + kept], c[pos:pos + kept])
            pos += int(oc[w])
        # at the owner: rows and tags, slots past the count tagged -1
        rows = torch.empty(world * cap, dtype=torch.int32, device="cuda")
        tags = torch.empty(world * cap, dtype=torch.int32, device="cuda")
        capi.check(L.xb_unpack_routed_padded(ops.ptr(rec), world, cap, ops.ptr(rows), ops.ptr(tags), ops.stream()))
        tg = tags.cpu().numpy().reshape(world, cap)
        for w in range(world):
            kept = min(int(oc[w]), cap - 1)
            assert (tg[w, 0] == -1) and (tg[w, 1 + kept:] == -1).all() and (tg[w, 1:1 + kept] >= 0).all()


def test_sharded_puller_behind_the_embedding_operator_on_one_rank():
    """An Embedding operator whose tables are served by b200_sharded_sparse_puller (world of one rank), through the
    Predictor API, against the same operator on the plain HBM puller and against the oracle."""
    pkg.load()
    from x_deeplearning_b200 import blaze_api as api
    rng = np.random.default_rng(21)
    dim, B = 32, 700
    tables = {"ta": rng.normal(0, 0.1, (5000, dim)).astype(np.float16).astype(np.float32),
              "tb": rng.normal(0, 0.1, (800, dim)).astype(np.float16).astype(np.float32)}
    groups = [("g0", "ta"), ("g1", "ta"), ("g2", "ta"), ("g3", "tb"), ("g4", "tb")]
    conf = "".join('feature_group_config { feature_group: "%s" table_name: "%s" dim: %d }\n' % (g, t, dim) for g, t in groups)
    conf += "block_config {\n" + "".join('  embedding_block_config_item { feature_group: "%s" udf_type: 0 }\n' % g for g, _ in groups) + "}\n"
    ins, feeds = [], {}
    for g, t in groups:
        counts = rng.integers(0, 12, B).astype(np.int32)
        ids = rng.integers(0, len(tables[t]), int(counts.sum())).astype(np.int64)
        feeds[g] = (ids, counts)
        ins += [g + ".ids", g + ".values", g + ".segments"]
    text = api.netdef_text([api.op_text("Embedding", ins, ["out"], {"embedding_config": conf})],
                           [(n, 10 if n.endswith(".ids") else 2 if n.endswith(".segments") else 12) for n in ins], [("out", 12)])
    results = []
    for sharded_puller in (False, True):
        mgr = api.PredictorManager()
        if sharded_puller:
            mgr.init_sharded(0, 1, None, max_ids_per_step=B * 12 * len(groups), partial_dtype=1)
        else:
            mgr.load_sparse(None, "b200_sparse_puller")
        for t, w in tables.items():
            mgr.add_table(t, w, 12)
        mgr.load_model_text(text)
        p = mgr.create_predictor()
        keep = []
        for g, (ids, counts) in feeds.items():
            keep += [p.feed(g + ".ids", ids), p.feed(g + ".values", np.ones(len(ids), np.float16)), p.feed(g + ".segments", counts)]
        p.forward()
        results.append(p.output("out").astype(np.float32))
        p.forward()                                            # the context and its buffers are reused
        np.testing.assert_array_equal(results[-1], p.output("out").astype(np.float32))
        p.close()
        mgr.close()
    np.testing.assert_array_equal(results[0], results[1])      # fp32 partial sums, one owner: the same bits
    want = np.zeros((B, len(groups) * dim), np.float32)
    for k, (g, t) in enumerate(groups):
        ids, counts = feeds[g]
        orc.embedding_pool(tables[t], ids, np.ones(len(ids), np.float32), counts, [dict(udf=0, out=want, col=k * dim)])
    np.testing.assert_allclose(results[1], want, rtol=2e-3, atol=2e-3)
