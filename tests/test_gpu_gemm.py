"""GEMM family: both engines through xb_gemm against the CPU oracle and the reference fixtures."""
import json
import os

import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
FIX = json.load(open(os.path.join(HERE, "golden", "blaze_op_fixtures.json")))


def _ops():
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    return ops, capi


def _status_ok(ops):
    torch.cuda.synchronize()
    assert ops.device_status() == 0, "a bounded wait ran out inside a tensor-core kernel"


@pytest.mark.parametrize("name", ["op/gemm/gemm_net_v1_cpu.conf"] +
                         ["fused_op/fused_parallel_gemm/fused_parallel_gemm_net_v%d_cpu.conf" % i for i in range(1, 6)])
def test_fp32_engine_reproduces_reference_fixtures(name):
    ops, capi = _ops()
    net = FIX[name]
    import oracle_net
    env = {}
    for op in net["ops"]:
        if op["type"] == "ConstantFill":
            env[op["output"][0]] = oracle_net.constant_fill(op)
    op = [o for o in net["ops"] if o["type"] != "ConstantFill"][0]
    A, B = [torch.from_numpy(env[n]).cuda() for n in op["input"][:2]]
    bias = torch.from_numpy(env[op["input"][2]]).cuda() if len(op["input"]) > 2 else None
    ta = bool(op["arg"].get("transA", {}).get("i", 0))
    tb = bool(op["arg"].get("transB", {}).get("i", 0))
    P = op["arg"].get("parallel_num", {}).get("i", 1)
    M, K = (A.shape[1], A.shape[0]) if ta else A.shape
    N = (B.shape[0] // P) if tb else B.shape[1]
    Y = torch.empty((P * M, N), device="cuda")
    ops.gemm(A, B, Y=Y, bias=bias, trans_a=ta, trans_b=tb, batch=P, M=M, N=N, K=K,
             strides=(0, K * N, N if bias is not None else 0, M * N), bias_kind=capi.XB_BIAS_ROW if bias is not None else None,
             engine=capi.XB_GEMM_SIMT)
    exp = net["expected"]["output"]
    want = np.array(exp["values"], np.float32).reshape(exp["shape"])
    np.testing.assert_allclose(Y.cpu().numpy(), want, rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_fp32_engine_random_with_epilogues(ta, tb):
    ops, capi = _ops()
    rng = np.random.default_rng(ta * 2 + tb)
    M, N, K = 77, 45, 131
    A = rng.normal(0, 1, (K, M) if ta else (M, K)).astype(np.float32)
    B = rng.normal(0, 0.2, (N, K) if tb else (K, N)).astype(np.float32)
    bias = rng.normal(0, 1, (M, N)).astype(np.float32)
    g, mu, var = rng.uniform(0, 0.5, N).astype(np.float32), rng.normal(0, 0.1, N).astype(np.float32), rng.uniform(0.5, 1.5, N).astype(np.float32)
    want = orc.dice(orc.gemm_op(A, B, bias, bool(ta), bool(tb), 0.7, 1.3), g, mu, var)
    c = lambda x: torch.from_numpy(x).cuda()
    Y = ops.gemm(c(A), c(B), bias=c(bias), trans_a=bool(ta), trans_b=bool(tb), alpha=0.7, beta=1.3,
                 epilogue=capi.XB_EPI_DICE, ep=(c(g), c(mu), c(var)), engine=capi.XB_GEMM_SIMT)
    np.testing.assert_allclose(Y.cpu().numpy(), want, rtol=2e-5, atol=2e-5)


def _tc_case(M, N, K, epi, rng, out_dtype=torch.float16, lda=None, bias_full=False):
    ops, capi = _ops()
    lda = lda or K
    A = (rng.normal(0, 1, (M, lda))).astype(np.float16)
    W = (rng.normal(0, 1 / np.sqrt(K), (K, N))).astype(np.float16)          # Blaze layout [K, N]
    bias = rng.normal(0, 0.5, (M, N) if bias_full else N).astype(np.float32)
    Af, Wf = A[:, :K].astype(np.float32), W.astype(np.float32)
    want = orc.gemm_op(Af, Wf, bias)
    c = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    kw = {}
    if epi == "dice":
        g, mu, var = rng.uniform(0, 0.5, N).astype(np.float32), rng.normal(0, 0.1, N).astype(np.float32), rng.uniform(0.5, 1.5, N).astype(np.float32)
        want = orc.dice(want, g, mu, var)
        kw = dict(epilogue=capi.XB_EPI_DICE, ep=(c(g), c(mu), c(var)))
    elif epi == "prelu":
        sl = rng.uniform(0.1, 0.4, N).astype(np.float32)
        want = orc.prelu(want, sl)
        kw = dict(epilogue=capi.XB_EPI_PRELU, ep=(c(sl), None, None), ep_count=N)
    elif epi == "sigmoid":
        want = orc.sigmoid(want)
        kw = dict(epilogue=capi.XB_EPI_SIGMOID)
    Wk = ops.pack_weight_kmajor(c(W), torch.float16)                          # [N, ldk]
    Y = torch.empty((M, N), dtype=out_dtype, device="cuda")
    dA = c(A)
    ops.gemm(dA, Wk, Y=Y, bias=c(bias), trans_b=True, M=M, N=N, K=K, lda=lda, engine=capi.XB_GEMM_TCGEN05, **kw)
    _status_ok(ops)
    got = Y.float().cpu().numpy()
    tol = 2e-3 if out_dtype == torch.float16 else 2e-4
    scale = np.abs(Af) @ np.abs(Wf) + np.abs(bias)
    err = np.abs(got - want)
    assert (err <= tol * (1 + scale)).all(), (float(err.max()), np.unravel_index(err.argmax(), err.shape))


@pytest.mark.parametrize("M,N,K,epi", [(128, 64, 64, "none"), (128, 16, 16, "none"), (300, 80, 144, "dice"),
                                       (1000, 200, 328, "dice"), (1000, 80, 200, "dice"), (513, 128, 256, "prelu"),
                                       (4096, 256, 512, "sigmoid"), (200, 1024, 1280, "prelu"), (77, 40, 80, "none")])
def test_tcgen05_engine_matches_oracle(M, N, K, epi):
    _tc_case(M, N, K, epi, np.random.default_rng(M + N + K))


def test_tcgen05_engine_fp32_output_full_bias_and_padded_lda():
    _tc_case(260, 48, 100, "none", np.random.default_rng(3), out_dtype=torch.float32, lda=104, bias_full=True)


@pytest.mark.parametrize("engine", ["tcgen05", "simt"])
@pytest.mark.parametrize("M,group,N,ks,kl,epi", [(600, 200, 200, 184, 144, "dice"), (96, 96, 80, 40, 72, "none"),
                                                 (1000, 1, 64, 16, 64, "prelu")])
def test_pruned_product_with_grouped_bias(engine, M, group, N, ks, kl, epi):
    """X1 x W1 computed once per row group (fp32), added in the epilogue of X2 x W2: the PrunedGemm form."""
    ops, capi = _ops()
    rng = np.random.default_rng(M + N + ks)
    m = M // group
    xs = rng.normal(0, 1, (m, ks)).astype(np.float16)
    xl = rng.normal(0, 1, (M, kl)).astype(np.float16)
    ws = rng.normal(0, 1 / np.sqrt(ks), (ks, N)).astype(np.float16)
    wl = rng.normal(0, 1 / np.sqrt(kl), (kl, N)).astype(np.float16)
    b = rng.normal(0, 0.3, N).astype(np.float32)
    f = lambda a: a.astype(np.float32)
    want = orc.pruned_gemm(f(xs), f(xl), f(ws), f(wl), b)
    c = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    kw = {}
    if epi == "dice":
        g, mu, var = rng.uniform(0, 0.5, N).astype(np.float32), rng.normal(0, 0.1, N).astype(np.float32), rng.uniform(0.5, 1.5, N).astype(np.float32)
        want = orc.dice(want, g, mu, var)
        kw = dict(epilogue=capi.XB_EPI_DICE, ep=(c(g), c(mu), c(var)))
    elif epi == "prelu":
        sl = rng.uniform(0.1, 0.4, N).astype(np.float32)
        want = orc.prelu(want, sl)
        kw = dict(epilogue=capi.XB_EPI_PRELU, ep=(c(sl), None, None), ep_count=N)
    eng = capi.XB_GEMM_TCGEN05 if engine == "tcgen05" else capi.XB_GEMM_SIMT
    part = torch.empty((m, N), dtype=torch.float32, device="cuda")
    Y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    dxs, dxl = c(xs), c(xl)
    ops.gemm(dxs, ops.pack_weight_kmajor(c(ws), torch.float16), Y=part, bias=c(b), trans_b=True, M=m, N=N, K=ks, engine=eng)
    ops.gemm(dxl, ops.pack_weight_kmajor(c(wl), torch.float16), Y=Y, bias=part, bias_kind=capi.XB_BIAS_FULL, ldbias=N,
             bias_row_group=group, trans_b=True, M=M, N=N, K=kl, engine=eng, **kw)
    _status_ok(ops)
    got = Y.float().cpu().numpy()
    scale = np.abs(f(xs)) @ np.abs(f(ws))
    scale = np.repeat(scale, group, axis=0) + np.abs(f(xl)) @ np.abs(f(wl)) + np.abs(b)
    err = np.abs(got - want)
    assert (err <= 2e-3 * (1 + scale)).all(), float(err.max())


def test_parallel_gemm_benchmark_config():
    """8 branches of [4096,256]x[256,128] + bias + PReLU(0.25), fp16, concatenated to [4096,1024]."""
    ops, capi = _ops()
    from x_deeplearning_b200 import workloads
    cfg = workloads.parallel_gemm_config(0)
    P, M, K = cfg["A"].shape
    N = cfg["W"].shape[2]
    c = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    A, W, bias = c(cfg["A"]).half(), c(cfg["W"]).half(), c(cfg["bias"])
    slope = torch.full((1,), cfg["alpha"], device="cuda")
    Wk = ops.pack_weight_kmajor(W, torch.float16, batch=P)
    Y = torch.empty((M, P * N), dtype=torch.float16, device="cuda")
    ops.gemm(A, Wk, Y=Y, bias=bias, trans_b=True, batch=P, M=M, N=N, K=K, lda=K, ldb=K, ldy=P * N,
             strides=(M * K, N * K, N, N), bias_kind=capi.XB_BIAS_ROW, epilogue=capi.XB_EPI_PRELU,
             ep=(slope, None, None), ep_count=1, engine=capi.XB_GEMM_TCGEN05)
    _status_ok(ops)
    got = Y.float().cpu().numpy()
    for p in range(P):
        want = orc.prelu(orc.gemm_op(cfg["A"][p], cfg["W"][p], cfg["bias"][p]), np.array([cfg["alpha"]], np.float32))
        np.testing.assert_allclose(got[:, p * N:(p + 1) * N], want, rtol=2e-3, atol=2e-3)
    # reference layout: one shared input, branches stacked on axis 0 (FusedParallelGemm)
    Y0 = torch.empty((P * M, N), dtype=torch.float16, device="cuda")
    ops.gemm(A[0], Wk, Y=Y0, bias=bias, trans_b=True, batch=P, M=M, N=N, K=K, lda=K, ldb=K, ldy=N,
             strides=(0, N * K, N, M * N), bias_kind=capi.XB_BIAS_ROW, engine=capi.XB_GEMM_TCGEN05)
    _status_ok(ops)
    want0 = orc.fused_parallel_gemm(cfg["A"][0], cfg["W"].reshape(P * K, N), cfg["bias"].reshape(-1), P)
    np.testing.assert_allclose(Y0.float().cpu().numpy(), want0, rtol=2e-3, atol=2e-3)


def test_tcgen05_engine_resident_weight_tile_runs():
    """Many m tiles per weight tile and several tiles per CTA: the weight tile stays in shared memory while a
    CTA walks a contiguous run of tiles, and is replaced when the run crosses into the next n tile or batch
    entry. Ragged in every direction: last m tile 77 rows, last n tile 64 columns, last k block 8 wide."""
    ops, capi = _ops()
    rng = np.random.default_rng(12)
    P, M, N, K = 3, 5197, 320, 200
    A = rng.normal(0, 1, (P, M, K)).astype(np.float16)
    W = (rng.normal(0, 1, (P, K, N)) / np.sqrt(K)).astype(np.float16)
    bias = rng.normal(0, 0.1, (P, N)).astype(np.float32)
    c = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    Wk = ops.pack_weight_kmajor(c(W), torch.float16, batch=P)
    ldk = Wk.shape[-1]
    slope = torch.full((1,), 0.25, device="cuda")
    Y = torch.zeros((P, M, N), dtype=torch.float16, device="cuda")
    ops.gemm(c(A), Wk, Y=Y, bias=c(bias), trans_b=True, batch=P, M=M, N=N, K=K, lda=K, ldb=ldk, ldy=N,
             strides=(M * K, N * ldk, N, M * N), bias_kind=capi.XB_BIAS_ROW, epilogue=capi.XB_EPI_PRELU,
             ep=(slope, None, None), ep_count=1, engine=capi.XB_GEMM_TCGEN05)
    _status_ok(ops)
    got = Y.float().cpu().numpy()
    for p in range(P):
        want = orc.prelu(orc.gemm_op(A[p].astype(np.float32), W[p].astype(np.float32), bias[p]), np.array([0.25], np.float32))
        np.testing.assert_allclose(got[p], want, rtol=2e-3, atol=2e-3)


def test_auto_engine_falls_back_for_layouts_tma_cannot_take():
    ops, capi = _ops()
    rng = np.random.default_rng(5)
    A = torch.from_numpy(rng.normal(0, 1, (50, 324)).astype(np.float16)).cuda()      # lda 324 is not a multiple of 8
    W = torch.from_numpy(rng.normal(0, 0.05, (324, 30)).astype(np.float16)).cuda()
    Y = ops.gemm(A, W)
    want = orc.gemm_op(A.float().cpu().numpy(), W.float().cpu().numpy())
    np.testing.assert_allclose(Y.float().cpu().numpy(), want, rtol=2e-3, atol=2e-3)
    with pytest.raises(capi.XbError, match="tcgen05 engine needs"):
        ops.gemm(A, W, engine=capi.XB_GEMM_TCGEN05)
