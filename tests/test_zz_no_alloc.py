"""xb_embedding_pool_static: the pooling entry point for callers that cannot allocate
(operators living inside a fixed memory plan). It must give exactly what
xb_embedding_pool gives with caller-provided scratch, call after call, although all
calls share one built-in scratch array that still holds the previous call's offsets.

Collected last on purpose (file name), so that a run that stops at the first failure
has already been through every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu


def _items(capi, dim, out):
    return [dict(udf=capi.XB_UDF_SUM, out=out, col=0), dict(udf=capi.XB_UDF_AVG, out=out, col=dim),
            dict(udf=capi.XB_UDF_ASSIGN, trunc_dir=capi.XB_TRUNC_REVERSE, trunc_num=3, out=out, col=2 * dim)]


def _groups(ops, capi, table, rng, batch, max_len, out, host=None):
    counts = rng.integers(0, max_len + 1, batch).astype(np.int32)
    n = int(counts.sum())
    ids_h = rng.integers(0, table.rows, n).astype(np.int64)
    vals_h = rng.normal(1, 0.3, n).astype(np.float32)
    if host is not None:
        host.update(ids=ids_h, values=vals_h, counts=counts)
    ids = torch.from_numpy(ids_h).cuda()
    vals = torch.from_numpy(vals_h).cuda()
    seg = torch.from_numpy(counts).cuda()                     # counts, so the call needs offset scratch
    return [ops.make_group(table, ids, vals, seg, _items(capi, table.dim, out), torch.float32)]


def test_static_scratch_entry_point_matches_the_allocating_one_twice():
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    L = capi.lib()
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.5, (4000, 18)).astype(np.float32)
    table = ops.Table(torch.from_numpy(w), torch.float32)
    width = 18 * 5
    # two calls in a row with different batch sizes: the second finds the first one's offsets in the array
    for batch, max_len in ((700, 9), (333, 40)):
        want = torch.full((batch, width), 5.0, device="cuda")
        got = torch.full((batch, width), 5.0, device="cuda")
        state = rng.bit_generator.state
        host = {}
        gw = _groups(ops, capi, table, rng, batch, max_len, want, host)
        rng.bit_generator.state = state                       # same ids for both entry points
        gg = _groups(ops, capi, table, rng, batch, max_len, got)
        ops.embedding_pool(gw)
        arr = (capi.PoolGroup * 1)(*gg)
        capi.check(L.xb_embedding_pool_static(arr, 1, ops.stream()))
        torch.cuda.synchronize()
        assert torch.equal(got, want)                          # same kernels, same order: bit-identical
        assert float(want.abs().sum()) > 0
        # and against the CPU oracle (fp32 pooled sums: 1e-5 relative to the sum of magnitudes)
        ref = np.full((batch, width), 5.0, np.float32)
        mag = np.full((batch, width), 5.0, np.float32)
        orc.embedding_pool(w, host["ids"], host["values"], host["counts"], _items(capi, 18, ref))
        orc.embedding_pool(np.abs(w), host["ids"], np.abs(host["values"]), host["counts"], _items(capi, 18, mag))
        err = np.abs(got.cpu().numpy() - ref)
        assert (err <= 1e-5 * np.maximum(mag, 1e-3) + 1e-7).all(), float(err.max())


def test_static_scratch_limit_is_the_scratch_bytes_function_over_several_groups():
    """Several groups that pass counts: accepted just under the limit that xb_embedding_pool_scratch_bytes
    computes (offsets AND scan partial sums of every group), rejected just over it."""
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    L = capi.lib()
    limit = int(L.xb_embedding_pool_static_max_bytes())
    table = ops.Table(torch.ones(8, 4), torch.float32)
    n_groups = 4

    def call(batch):
        outs = [torch.full((batch, 4), 7.0, device="cuda") for _ in range(n_groups)]
        seg = torch.ones(batch, dtype=torch.int32, device="cuda")
        ids = torch.zeros(batch, dtype=torch.int64, device="cuda")
        gs = [ops.make_group(table, ids, None, seg, [dict(udf=capi.XB_UDF_SUM, out=o)], torch.float32) for o in outs]
        arr = (capi.PoolGroup * n_groups)(*gs)
        need = int(L.xb_embedding_pool_scratch_bytes(arr, n_groups))
        rc = L.xb_embedding_pool_static(arr, n_groups, ops.stream())
        torch.cuda.synchronize()
        return need, rc, outs

    # largest batch whose four groups fit: 4*(batch+1) rounded to 256, plus 256 of scan sums, per group
    per_group = limit // n_groups
    fit = (per_group - 256) // 4 - 1
    need, rc, outs = call(fit)
    assert need <= limit and rc == 0, (need, rc)
    for o in outs:
        assert torch.equal(o, torch.ones_like(o))               # one id per sample, row of ones
    need, rc, _ = call(fit + 64)
    assert need > limit and rc == -5, (need, rc)
    # sizing by the offsets alone would have let this one through
    assert n_groups * 4 * (fit + 64 + 1) <= limit


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    L = capi.lib()
    limit = int(L.xb_embedding_pool_static_max_bytes())
    assert limit == 1 << 20
    batch = limit // 4 + 10                                   # 4*(batch+1) bytes of offsets > the built-in array
    table = ops.Table(torch.zeros(8, 4), torch.float32)
    out = torch.zeros((batch, 4), device="cuda")
    seg = torch.zeros(batch, dtype=torch.int32, device="cuda")
    ids = torch.zeros(1, dtype=torch.int64, device="cuda")
    g = ops.make_group(table, ids, None, seg, [dict(udf=capi.XB_UDF_SUM, out=out)], torch.float32)
    g.n_ids = 0
    arr = (capi.PoolGroup * 1)(g)
    assert L.xb_embedding_pool_static(arr, 1, ops.stream()) == -5
    assert b"built-in buffer holds" in L.xb_last_error()
    # the same groups with exclusive offsets need no scratch and are accepted
    off = torch.zeros(batch + 1, dtype=torch.int32, device="cuda")
    g2 = ops.make_group(table, ids, None, off, [dict(udf=capi.XB_UDF_SUM, out=out)], torch.float32,
                        segments_are_offsets=True)
    g2.n_ids = 0
    arr2 = (capi.PoolGroup * 1)(g2)
    capi.check(L.xb_embedding_pool_static(arr2, 1, ops.stream()))
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
