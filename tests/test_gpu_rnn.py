"""GRU / AUGRU kernels against the CPU oracle (GRU pinned by the reference fixtures, AUGRU unpinned)."""
import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu


def _ops():
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    return ops, capi, capi.lib()


@pytest.mark.parametrize("B,T,H,dtype,tol", [(1000, 100, 36, torch.float32, 2e-5), (7, 5, 64, torch.float32, 2e-5),
                                              (33, 20, 36, torch.float16, 4e-3), (3, 1, 1, torch.float32, 1e-6)])
def test_gru_matches_oracle(B, T, H, dtype, tol):
    ops, capi, L = _ops()
    rng = np.random.default_rng(B + T + H)
    r = lambda a: torch.from_numpy(a.astype(np.float32)).to("cuda", dtype)
    x = rng.normal(0, 1, (B, T, H))
    x[: B // 3, : T // 2] = 0                      # leading padding steps
    Wi, Wh = rng.normal(0, 1 / np.sqrt(H), (H, 3 * H)), rng.normal(0, 1 / np.sqrt(H), (H, 3 * H))
    bi, bh = rng.normal(0, 0.1, 3 * H), rng.normal(0, 0.1, 3 * H)
    dx, dWi, dWh, dbi, dbh = r(x), r(Wi), r(Wh), r(bi), r(bh)
    y = torch.empty_like(dx)
    capi.check(L.xb_gru(ops.ptr(dx), ops.ptr(y), B, T, H, ops.ptr(dWi), ops.ptr(dWh), ops.ptr(dbi), ops.ptr(dbh),
                        ops.dt(dx), ops.stream()))
    f = lambda t: t.float().cpu().numpy()
    want = orc.gru(f(dx), f(dWh), f(dWi), f(dbh), f(dbi))
    np.testing.assert_allclose(f(y), want, rtol=tol, atol=tol)
    if B >= 3 and T >= 2:
        assert (f(y)[0, : T // 2] == 0).all()


@pytest.mark.parametrize("B,T,H,dtype,tol", [(1000, 100, 36, torch.float32, 2e-5), (5, 9, 16, torch.float16, 4e-3)])
def test_augru_matches_oracle(B, T, H, dtype, tol):
    ops, capi, L = _ops()
    rng = np.random.default_rng(B + H)
    r = lambda a: torch.from_numpy(a.astype(np.float32)).to("cuda", dtype)
    x, att = rng.normal(0, 1, (B, T, H)), rng.uniform(0, 1, (B, T))
    Wg, bg = rng.normal(0, 1 / np.sqrt(2 * H), (2 * H, 2 * H)), rng.normal(0, 0.1, 2 * H)
    Wc, bc = rng.normal(0, 1 / np.sqrt(2 * H), (2 * H, H)), rng.normal(0, 0.1, H)
    dx, da, dWg, dbg, dWc, dbc = r(x), r(att), r(Wg), r(bg), r(Wc), r(bc)
    y = torch.empty_like(dx)
    capi.check(L.xb_augru(ops.ptr(dx), ops.ptr(da), ops.ptr(y), B, T, H, ops.ptr(dWg), ops.ptr(dbg), ops.ptr(dWc),
                          ops.ptr(dbc), ops.dt(dx), ops.stream()))
    f = lambda t: t.float().cpu().numpy()
    want = orc.augru(f(dx), f(da), f(dWg), f(dbg), f(dWc), f(dbc))
    np.testing.assert_allclose(f(y), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("engine", ["simt", "tc"])
@pytest.mark.parametrize("R,n_cand,T,H", [(2, 300, 100, 36), (3, 130, 7, 36), (1, 5, 1, 20)])
def test_augru_over_a_shared_sequence_matches_oracle(engine, R, n_cand, T, H):
    """xb_augru_shared: every candidate of a request walks the request's sequence with its own scores; only the final
    state is kept. The tcgen05 engine keeps the state in fp32 and rounds it to fp16 as an MMA operand each step."""
    ops, capi, L = _ops()
    rng = np.random.default_rng(R * 1000 + n_cand + T)
    h16 = lambda a: torch.from_numpy(a.astype(np.float32)).to("cuda", torch.float16)
    x, att = rng.normal(0, 0.7, (R, T, H)), rng.dirichlet(np.ones(T) * 0.3, R * n_cand)      # softmax-like scores
    Wg, bg = rng.normal(0, 1 / np.sqrt(2 * H), (2 * H, 2 * H)), rng.normal(0.5, 0.2, 2 * H)
    Wc, bc = rng.normal(0, 1 / np.sqrt(2 * H), (2 * H, H)), rng.normal(0, 0.1, H)
    dx, da, dWg, dbg, dWc, dbc = h16(x), h16(att), h16(Wg), h16(bg), h16(Wc), h16(bc)
    y = torch.full((R * n_cand, H), 9.0, dtype=torch.float16, device="cuda")
    eng = capi.XB_GEMM_SIMT if engine == "simt" else capi.XB_GEMM_TCGEN05
    capi.check(L.xb_augru_shared(ops.ptr(dx), ops.ptr(da), ops.ptr(y), R, n_cand, T, H, ops.ptr(dWg), ops.ptr(dbg),
                                 ops.ptr(dWc), ops.ptr(dbc), eng, ops.stream()))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    f = lambda t: t.float().cpu().numpy()
    xs = np.repeat(f(dx), n_cand, axis=0)                                       # [R * n_cand, T, H]
    want = orc.augru(xs, f(da), f(dWg), f(dbg), f(dWc), f(dbc))[:, T - 1, :]
    tol = 4e-3 if engine == "simt" else 8e-3
    np.testing.assert_allclose(f(y), want, rtol=0, atol=tol)


def test_augru_tcgen05_engine_declines_shapes_without_selector_slots():
    ops, capi, L = _ops()
    z = torch.zeros(64 * 64 * 4, dtype=torch.float16, device="cuda")
    rc = L.xb_augru_shared(ops.ptr(z), ops.ptr(z), ops.ptr(z), 1, 4, 3, 32, ops.ptr(z), ops.ptr(z), ops.ptr(z), ops.ptr(z),
                           capi.XB_GEMM_TCGEN05, ops.stream())
    assert rc == -2 and b"tcgen05 engine" in L.xb_last_error()
