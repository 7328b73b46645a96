"""Stand-alone operators against the oracle and the reference fixtures."""
import ctypes as C
import json
import os

import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu


def _l():
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    return ops, capi, capi.lib()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.float16, 2e-3)])
def test_activations(dtype, tol):
    ops, capi, L = _l()
    rng = np.random.default_rng(0)
    x = rng.normal(0, 2, (37, 80)).astype(np.float32)
    g, mu, var = rng.uniform(0, 0.5, 80).astype(np.float32), rng.normal(0, 0.1, 80).astype(np.float32), rng.uniform(0.5, 1.5, 80).astype(np.float32)
    c = lambda a: torch.from_numpy(a).to("cuda", dtype)
    r = lambda a: c(a).float().cpu().numpy()
    dx, y = c(x), torch.empty((37, 80), dtype=dtype, device="cuda")
    dg, dmu, dvar = c(g), c(mu), c(var)          # keep the device tensors alive while their pointers are in use
    s, dt = ops.stream(), ops.dt(dx)
    capi.check(L.xb_dice(ops.ptr(dx), ops.ptr(y), 37, 80, ops.ptr(dg), ops.ptr(dmu), ops.ptr(dvar), 0, dt, s))
    np.testing.assert_allclose(y.float().cpu().numpy(), orc.dice(r(x), r(g), r(mu), r(var)), rtol=tol, atol=tol)
    w = c(g)
    capi.check(L.xb_prelu(ops.ptr(dx), ops.ptr(y), 37 * 80, ops.ptr(w), 80, dt, dt, s))
    np.testing.assert_allclose(y.float().cpu().numpy(), orc.prelu(r(x), r(g)), rtol=tol, atol=tol)
    capi.check(L.xb_sigmoid(ops.ptr(dx), ops.ptr(y), 37 * 80, dt, s))
    np.testing.assert_allclose(y.float().cpu().numpy(), orc.sigmoid(r(x)), rtol=tol, atol=tol)
    capi.check(L.xb_softmax(ops.ptr(dx), ops.ptr(y), 37, 80, 1, dt, s))
    np.testing.assert_allclose(y.float().cpu().numpy(), orc.softmax(r(x), 1), rtol=tol * 5, atol=tol)
    capi.check(L.xb_batchnorm(ops.ptr(dx), ops.ptr(y), 37 * 80, 80, ops.ptr(dg), ops.ptr(dmu), ops.ptr(dmu),
                              ops.ptr(dvar), 0.001, 0, dt, s))
    np.testing.assert_allclose(y.float().cpu().numpy(), orc.batchnorm(r(x), r(g), r(mu), r(mu), r(var)), rtol=tol * 5, atol=tol * 5)


def test_softmax_inner_axis_and_reduce_sum_and_copy():
    ops, capi, L = _l()
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, (3, 5, 4)).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    y = torch.empty_like(dx)
    capi.check(L.xb_softmax(ops.ptr(dx), ops.ptr(y), 3, 5, 4, capi.XB_F32, ops.stream()))
    np.testing.assert_allclose(y.cpu().numpy(), orc.softmax(x, 1), rtol=1e-5, atol=1e-6)
    z = torch.empty((3, 4), device="cuda")
    capi.check(L.xb_reduce_sum(ops.ptr(dx), ops.ptr(z), 3, 5, 4, capi.XB_F32, ops.stream()))
    np.testing.assert_allclose(z.cpu().numpy(), x.sum(1), rtol=1e-6, atol=1e-6)
    # Fuse: a 1-row tensor broadcast in front of an M-row tensor
    x1 = torch.from_numpy(rng.normal(0, 1, (1, 6)).astype(np.float32)).cuda()
    x2 = torch.from_numpy(rng.normal(0, 1, (9, 3)).astype(np.float32)).cuda()
    out = torch.empty((9, 9), device="cuda")
    capi.check(L.xb_copy2d(ops.ptr(x1), 0, capi.XB_F32, ops.ptr(out), 9, capi.XB_F32, 9, 6, ops.stream()))
    capi.check(L.xb_copy2d(ops.ptr(x2), 3, capi.XB_F32, C.c_void_p(out.data_ptr() + 24), 9, capi.XB_F32, 9, 3, ops.stream()))
    np.testing.assert_array_equal(out.cpu().numpy(), orc.fuse(x1.cpu().numpy(), x2.cpu().numpy()))


def test_elementwise_broadcast():
    ops, capi, L = _l()
    rng = np.random.default_rng(2)
    a = rng.normal(0, 1, (2, 3, 1)).astype(np.float32)
    b = rng.normal(0, 1, (2,)).astype(np.float32)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    y = torch.empty((2, 3, 2), device="cuda")
    arr = lambda v: (C.c_int64 * 4)(*v)
    for op, f in ((capi.XB_EW_MUL, np.multiply), (capi.XB_EW_SUB, np.subtract), (capi.XB_EW_MAX, np.maximum)):
        capi.check(L.xb_elementwise(op, ops.ptr(da), arr([0, 3, 1, 0]), ops.ptr(db), arr([0, 0, 0, 1]), None, None,
                                    ops.ptr(y), arr([1, 2, 3, 2]), capi.XB_F32, ops.stream()))
        np.testing.assert_array_equal(y.cpu().numpy(), f(a, b))


def test_copy_segments_moves_every_range_in_one_launch():
    """Flat copies of odd lengths and alignments (id lists, counts, fp16 rows) against numpy slicing."""
    pkg.load()
    from x_deeplearning_b200 import capi, ops
    rng = np.random.default_rng(9)
    src = torch.from_numpy(rng.integers(0, 256, 3_000_000, dtype=np.uint8)).cuda()
    dst = torch.zeros(3_200_000, dtype=torch.uint8, device="cuda")
    want = np.zeros(3_200_000, np.uint8)
    host = src.cpu().numpy()
    lengths = [0, 1, 7, 16, 33, 800, 4096, 32 * 1024, 32 * 1024 + 1, 100_003, 1_000_000]
    items, so, do = [], 5, 3                                       # odd starts: the byte path
    for i, n in enumerate(lengths):
        if i % 2:                                                  # every other copy 16-byte aligned at both ends
            so, do = (so + 15) // 16 * 16, (do + 15) // 16 * 16
        items.append((src.data_ptr() + so, dst.data_ptr() + do, n))
        want[do:do + n] = host[so:so + n]
        so += n + 3
        do += n + 5
    table = torch.tensor([[a, b, n] for a, b, n in items], dtype=torch.int64).cuda()
    capi.check(capi.lib().xb_copy_segments(table.data_ptr(), len(items), max(lengths), ops.stream()))
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), want)
    # nothing to do
    capi.check(capi.lib().xb_copy_segments(None, 0, 0, ops.stream()))
