"""Embedding pooling: CUDA kernel (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu


def _run_case(rng, rows, dim, batch, max_len, tdtype, out_dtype, hashed, use_offsets, id32=False, miss=0.1,
              with_values=True, missing_table=False):
    m = pkg.load()
    from x_deeplearning_b200 import ops, capi
    w = rng.normal(0, 0.5, (rows, dim)).astype(np.float32)
    if tdtype == torch.float16:
        w = w.astype(np.float16).astype(np.float32)
    tkeys = rng.choice(1 << 30 if id32 else 1 << 40, size=rows, replace=False).astype(np.int64) if hashed else None
    counts = rng.integers(0, max_len + 1, batch).astype(np.int32)
    n = int(counts.sum())
    base = tkeys if hashed else np.arange(rows, dtype=np.int64)
    ids = base[rng.integers(0, rows, n)]
    bad = rng.random(n) < miss
    ids[bad] = (1 << 30) + 12345 if id32 else rng.integers(1 << 41, 1 << 42, int(bad.sum()))
    values = rng.normal(1, 0.5, n).astype(np.float32) if with_values else np.ones(n, np.float32)
    tn = 4
    width = 2 * dim + 2 * dim * tn + 3          # odd width: unaligned item offsets
    def items(out):
        return [dict(udf=0, out=out, col=1), dict(udf=1, out=out, col=1 + dim),
                dict(udf=2, trunc_dir=0, trunc_num=tn, out=out, col=2 + 2 * dim),
                dict(udf=2, trunc_dir=1, trunc_num=tn, out=out, col=2 + 2 * dim + dim * tn)]
    want = np.full((batch, width), 3.0, np.float32)
    scale = np.full((batch, width), 3.0, np.float32)
    if missing_table:
        for it in items(want):
            span = dim * (tn if it["udf"] == 2 else 1)
            want[:, it["col"]:it["col"] + span] = 0
        scale[:] = 1
    else:
        orc.embedding_pool(w, ids, values, counts, items(want), table_keys=tkeys)
        orc.embedding_pool(np.abs(w), ids, np.abs(values), counts, items(scale), table_keys=tkeys)
    dev = "cuda"
    table = None if missing_table else ops.Table(torch.from_numpy(w), tdtype, keys=None if tkeys is None else torch.from_numpy(tkeys))
    got = torch.full((batch, width), 3.0, dtype=out_dtype, device=dev)
    d_ids = torch.from_numpy(ids.astype(np.int32) if id32 else ids).to(dev)
    d_val = torch.from_numpy(values).to(dev) if with_values else None
    if use_offsets:
        off = np.zeros(batch + 1, np.int32)
        np.cumsum(counts, out=off[1:])
        seg = torch.from_numpy(off).to(dev)
    else:
        seg = torch.from_numpy(counts).to(dev)
    g = ops.make_group(table, d_ids, d_val, seg, items(got), out_dtype, segments_are_offsets=use_offsets, dim=dim)
    ops.embedding_pool([g])
    torch.cuda.synchronize()
    got = got.float().cpu().numpy()
    tol = 1e-5 if out_dtype == torch.float32 else 1.5e-3
    err = np.abs(got - want)
    assert (err <= tol * np.maximum(scale, 1e-3) + 1e-7).all(), float((err / np.maximum(scale, 1e-3)).max())
    # columns outside every item keep the caller's fill value
    assert (got[:, 0] == 3.0).all() and (got[:, -1] == 3.0).all()


@pytest.mark.parametrize("dim,tdtype", [(16, torch.float32), (18, torch.float16), (32, torch.float16),
                                        (4, torch.float32), (1, torch.float32), (64, torch.float16),
                                        (36, torch.float32), (7, torch.float16)])
def test_pool_matches_oracle(dim, tdtype):
    rng = np.random.default_rng(dim)
    _run_case(rng, 3000, dim, 257, 13, tdtype, torch.float32, hashed=True, use_offsets=False)


@pytest.mark.parametrize("max_len", [1, 2, 50, 200])
def test_pool_segment_length_classes(max_len):
    rng = np.random.default_rng(100 + max_len)
    _run_case(rng, 2000, 16, 300, max_len, torch.float32, torch.float32, hashed=False, use_offsets=True)


def test_pool_fp16_output_int32_ids_and_unit_values():
    rng = np.random.default_rng(7)
    _run_case(rng, 1000, 18, 129, 9, torch.float16, torch.float16, hashed=True, use_offsets=False, id32=True,
              with_values=False)


def test_pool_missing_table_zero_fills():
    rng = np.random.default_rng(8)
    _run_case(rng, 100, 18, 65, 5, torch.float16, torch.float32, hashed=False, use_offsets=False, missing_table=True)


def _run_single_item(rng, rows, dim, batch, max_len, tdtype, out_dtype, udf, trunc_dir=0, hashed=False, id32=False,
                     with_values=True, use_offsets=True, min_len=0):
    """One item per feature group: the case the specialised kernels (static teams for small batches and
    kAssign, a per-warp segment queue for large sum / average batches) take."""
    pkg.load()
    from x_deeplearning_b200 import ops
    w = rng.normal(0, 0.5, (rows, dim)).astype(np.float32)
    if tdtype == torch.float16:
        w = w.astype(np.float16).astype(np.float32)
    tkeys = rng.choice(1 << 30 if id32 else 1 << 40, size=rows, replace=False).astype(np.int64) if hashed else None
    counts = rng.integers(min_len, max_len + 1, batch).astype(np.int32)
    n = int(counts.sum())
    base = tkeys if hashed else np.arange(rows, dtype=np.int64)
    ids = base[rng.integers(0, rows, n)]
    bad = rng.random(n) < 0.05
    ids[bad] = (1 << 30) + 12345 if id32 else rng.integers(1 << 41, 1 << 42, int(bad.sum()))
    values = rng.normal(1, 0.5, n).astype(np.float32) if with_values else np.ones(n, np.float32)
    tn = 5
    span = dim * (tn if udf == 2 else 1)
    width = span + 3

    def items(out):
        return [dict(udf=udf, trunc_dir=trunc_dir, trunc_num=tn, out=out, col=1)]
    want = np.full((batch, width), 3.0, np.float32)
    scale = np.full((batch, width), 3.0, np.float32)
    orc.embedding_pool(w, ids, values, counts, items(want), table_keys=tkeys)
    orc.embedding_pool(np.abs(w), ids, np.abs(values), counts, items(scale), table_keys=tkeys)
    table = ops.Table(torch.from_numpy(w), tdtype, keys=None if tkeys is None else torch.from_numpy(tkeys))
    got = torch.full((batch, width), 3.0, dtype=out_dtype, device="cuda")
    d_ids = torch.from_numpy(ids.astype(np.int32) if id32 else ids).cuda()
    d_val = torch.from_numpy(values).cuda() if with_values else None
    if use_offsets:
        off = np.zeros(batch + 1, np.int32)
        np.cumsum(counts, out=off[1:])
        seg = torch.from_numpy(off).cuda()
    else:
        seg = torch.from_numpy(counts).cuda()
    g = ops.make_group(table, d_ids, d_val, seg, items(got), out_dtype, segments_are_offsets=use_offsets, dim=dim)
    ops.embedding_pool([g])
    torch.cuda.synchronize()
    got = got.float().cpu().numpy()
    tol = 1e-5 if out_dtype == torch.float32 else 1.5e-3
    err = np.abs(got - want)
    assert (err <= tol * np.maximum(scale, 1e-3) + 1e-7).all(), float((err / np.maximum(scale, 1e-3)).max())
    assert (got[:, 0] == 3.0).all() and (got[:, -1] == 3.0).all()


@pytest.mark.parametrize("udf,trunc_dir", [(0, 0), (1, 0), (2, 0), (2, 1)])
@pytest.mark.parametrize("dim,tdtype,out_dtype", [(16, torch.float32, torch.float32), (18, torch.float16, torch.float16),
                                                  (36, torch.float16, torch.float32), (5, torch.float32, torch.float16),
                                                  (100, torch.float16, torch.float32)])
def test_pool_single_item_small_batch(udf, trunc_dir, dim, tdtype, out_dtype):
    rng = np.random.default_rng(1000 + 10 * dim + udf + trunc_dir)
    _run_single_item(rng, 3000, dim, 333, 11, tdtype, out_dtype, udf, trunc_dir, hashed=dim % 2 == 0)


@pytest.mark.parametrize("udf", [0, 1])
@pytest.mark.parametrize("dim,tdtype,out_dtype,max_len", [(16, torch.float32, torch.float32, 50),
                                                          (18, torch.float16, torch.float16, 7),
                                                          (36, torch.float16, torch.float32, 20),
                                                          (3, torch.float32, torch.float32, 9),
                                                          (72, torch.float32, torch.float32, 12)])
def test_pool_single_item_large_batch_segment_queue(udf, dim, tdtype, out_dtype, max_len):
    """Batches large enough for the segment-queue kernel, empty segments and missing keys included."""
    rng = np.random.default_rng(2000 + 10 * dim + udf)
    _run_single_item(rng, 5000, dim, 60001, max_len, tdtype, out_dtype, udf, hashed=dim == 36, use_offsets=dim != 18,
                     with_values=dim != 3, id32=dim == 3)


@pytest.mark.parametrize("udf", [0, 1])
@pytest.mark.parametrize("dim,tdtype,out_dtype,max_len", [(32, torch.float16, torch.float16, 3),
                                                          (16, torch.float32, torch.float32, 2),
                                                          (18, torch.float16, torch.float32, 4),
                                                          (3, torch.float32, torch.float16, 1),
                                                          (100, torch.float16, torch.float32, 3)])
def test_pool_very_short_segments_large_batch(udf, dim, tdtype, out_dtype, max_len):
    """Fewer than three ids per segment on average in a large call: the short-segment kernel; empty segments,
    missing keys, hashed and identity tables, counts and offsets, int32 ids, per-id values."""
    rng = np.random.default_rng(2500 + 10 * dim + udf)
    _run_single_item(rng, 5000, dim, 70003, max_len, tdtype, out_dtype, udf, hashed=dim == 18, use_offsets=dim != 16,
                     with_values=dim != 3, id32=dim == 3)


def test_pool_single_item_long_segments_few_samples():
    rng = np.random.default_rng(3000)
    _run_single_item(rng, 4000, 16, 9, 700, torch.float32, torch.float32, 0, min_len=300)
    _run_single_item(rng, 4000, 18, 5, 300, torch.float16, torch.float32, 2, trunc_dir=1, min_len=1)


def test_pool_rejects_bad_arguments():
    m = pkg.load()
    from x_deeplearning_b200 import ops, capi
    t = ops.Table(torch.zeros(4, 8), torch.float32)
    out = torch.zeros((2, 8), device="cuda")
    ids = torch.zeros(2, dtype=torch.int64, device="cuda")
    seg = torch.ones(2, dtype=torch.int32, device="cuda")
    g = ops.make_group(t, ids, None, seg, [dict(udf=7, out=out)], torch.float32)
    with pytest.raises(capi.XbError, match="Unsupported udf type"):
        ops.embedding_pool([g])
    g = ops.make_group(t, ids, None, seg, [dict(udf=0, out=out)], torch.float32, dim=4)
    g.dim = 4
    with pytest.raises(capi.XbError, match="dim"):
        ops.embedding_pool([g])


def test_pool_benchmark_config_full_size():
    """1M x 16 fp32 table, 512 x 20 segments, Zipf(1.1) ids, CSR offsets -> [512, 320]."""
    m = pkg.load()
    from x_deeplearning_b200 import ops, workloads
    cfg = workloads.embedding_config(seed=0)
    table = ops.Table(torch.from_numpy(cfg["table"]), torch.float32)
    want = np.zeros((512, 320), np.float32)
    got = torch.zeros((512, 320), device="cuda")
    groups = []
    for g, grp in enumerate(cfg["groups"]):
        orc.embedding_pool(cfg["table"], grp["ids"], grp["values"], grp["counts"], [dict(udf=0, out=want, col=16 * g)])
        groups.append(ops.make_group(table, torch.from_numpy(grp["ids"]).cuda(), torch.from_numpy(grp["values"]).cuda(),
                                     torch.from_numpy(grp["offsets"]).cuda(), [dict(udf=0, out=got, col=16 * g)],
                                     torch.float32, segments_are_offsets=True))
    ops.embedding_pool(groups)
    torch.cuda.synchronize()
    got = got.cpu().numpy()
    # |sum| <= 50 * 5 sigma: compare against the sum of magnitudes bound 50 * 0.05
    assert np.abs(got - want).max() <= 1e-5 * 2.5
    # size-independent property: pooling is linear in the per-id weights
    got2 = torch.zeros((512, 320), device="cuda")
    groups2 = []
    for g, grp in enumerate(cfg["groups"]):
        groups2.append(ops.make_group(table, torch.from_numpy(grp["ids"]).cuda(),
                                      torch.from_numpy(grp["values"] * 2).cuda(),
                                      torch.from_numpy(grp["offsets"]).cuda(), [dict(udf=0, out=got2, col=16 * g)],
                                      torch.float32, segments_are_offsets=True))
    ops.embedding_pool(groups2)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(got2.cpu().numpy(), 2 * got)       # scaling by 2 is exact in fp32


def test_gather_probe_runs_and_rejects_wide_rows():
    """The measurement aid touches every requested row and nothing else; rows wider than 64 bytes are refused."""
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    t = ops.Table(torch.randn(5000, 32), torch.float16)
    rows = torch.randint(0, 5000, (100_000,), dtype=torch.int32, device="cuda")
    sink = torch.zeros(1, device="cuda")
    ops.check(capi.lib().xb_gather_probe(t.desc, rows.data_ptr(), rows.numel(), sink.data_ptr(), ops.stream()))
    torch.cuda.synchronize()
    assert float(sink.item()) == 0.0 and ops.device_status() == 0
    wide = ops.Table(torch.randn(16, 64), torch.float32)
    with pytest.raises(capi.XbError, match="at most 64 bytes"):
        ops.check(capi.lib().xb_gather_probe(wide.desc, rows.data_ptr(), 16, sink.data_ptr(), ops.stream()))
