"""The C++ host runtime (Operator registry, Workspace, Net, Predictor, C API) on the GPU:
every reference operator fixture goes through PredictorManager / Predictor exactly as
the reference's TestOperatorOutput drives a text-proto NetDef
(blaze/blaze/test/operator/operator_test_common.h:19-84), with the net's device switched to CUDA."""
import json
import os

import numpy as np
import pytest

import pkg

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
FIX = json.load(open(os.path.join(HERE, "golden", "blaze_op_fixtures.json")))


def _api():
    pkg.load()
    from x_deeplearning_b200 import blaze_api
    return blaze_api


@pytest.mark.parametrize("name", sorted(FIX))
def test_reference_fixture_through_predictor(name):
    api = _api()
    net = FIX[name]
    mgr = api.PredictorManager()
    if "embedding" in name:
        mgr.load_sparse(None, "mock_sparse_puller")
    mgr.load_model_text(api.fixture_to_text(net))
    p = mgr.create_predictor(device_type=1, device_id=0)
    p.forward()
    for out, exp in net["expected"].items():
        got = p.output(out)
        want = np.array([float(str(v).rstrip("f")) for v in exp["values"]], np.float64).reshape(exp["shape"])
        assert list(got.shape) == list(exp["shape"]), (got.shape, exp["shape"])
        np.testing.assert_allclose(got.astype(np.float64), want, rtol=1e-5, atol=2e-6)
    p.close()
    mgr.close()


def test_errors_surface_like_blaze():
    api = _api()
    mgr = api.PredictorManager()
    with pytest.raises(api.BlazeError, match="parse NetDef text failed"):
        mgr.load_model_text('op { type: "Gemm" ')
    mgr.load_model_text(api.netdef_text([api.op_text("NoSuchOp", [], ["y"])], [], [("y", 1)]))
    with pytest.raises(api.BlazeError, match="NoSuchOp is not registered"):
        mgr.create_predictor()
    # CPU predictors do not exist in this backend
    mgr.load_model_text(api.netdef_text([api.constant_text("y", np.zeros(2), 1)], [], [("y", 1)]))
    with pytest.raises(api.BlazeError, match="CUDA devices only"):
        mgr.create_predictor(device_type=0)
    # shape errors raised inside an operator make Forward fail, not abort
    ops = [api.constant_text("a", np.zeros((2, 3)), 1), api.constant_text("b", np.zeros((4, 2)), 1),
           api.op_text("Gemm", ["a", "b"], ["y"])]
    mgr.load_model_text(api.netdef_text(ops, [], [("y", 1)]))
    p = mgr.create_predictor()
    with pytest.raises(api.BlazeError, match="a_k=3 b_k=4"):
        p.forward()
    p.close()
    mgr.close()


def test_fed_inputs_gemm_activation_fusion_and_shared_constants():
    api = _api()
    import orc
    rng = np.random.default_rng(0)
    M, K, N = 300, 144, 80
    W = rng.normal(0, 1 / 12, (K, N)).astype(np.float16)
    b = rng.normal(0, 0.1, N).astype(np.float16)
    g, mu, var = rng.uniform(0, 0.5, N).astype(np.float16), rng.normal(0, 0.1, N).astype(np.float16), rng.uniform(0.5, 1.5, N).astype(np.float16)
    ops = [api.constant_text("W", W, 12), api.constant_text("b", b, 12), api.constant_text("g", g, 12),
           api.constant_text("mu", mu, 12), api.constant_text("var", var, 12),
           api.op_text("Gemm", ["x", "W", "b"], ["h"]), api.op_text("Dice", ["h", "g", "mu", "var"], ["y"])]
    text = api.netdef_text(ops, [("x", 12)], [("y", 12)])
    f32 = lambda a: a.astype(np.float32)
    for optimize in (False, True):
        mgr = api.PredictorManager()
        mgr.load_model_text(text, optimize=optimize)
        preds = [mgr.create_predictor(), mgr.create_predictor()]          # share W, b, ... on the device
        for i, p in enumerate(preds):
            x = rng.normal(0, 1, (M + i, K)).astype(np.float16)
            keep = p.feed("x", x)
            p.forward()
            got = p.output("y")
            want = orc.dice(orc.gemm_op(f32(x), f32(W), f32(b)), f32(g), f32(mu), f32(var))
            np.testing.assert_allclose(got.astype(np.float32), want, rtol=3e-3, atol=3e-3)
            # fused: one kernel-library call (plus the one-off parameter conversions on the first run)
            p.forward()
            assert p.launches() == (1 if optimize else 2), p.launches()
            p.close()
        mgr.close()


@pytest.mark.parametrize("m1,m2", [(1, 300), (5, 1000), (260, 260), (400, 2)])
def test_pruned_gemm_operator_fp16_with_fused_dice(m1, m2):
    """PrunedGemm (blaze/blaze/operator/op/pruned_gemm_op.h): one-row broadcast as in the reference, row groups,
    equal row counts; with LoadModel's fusion pass folding the following Dice into the product."""
    api = _api()
    import orc
    rng = np.random.default_rng(m1 + m2)
    k1, k2, N = 184, 144, 200
    h = lambda a: a.astype(np.float16)
    W1, W2 = h(rng.normal(0, 1 / 14, (k1, N))), h(rng.normal(0, 1 / 12, (k2, N)))
    b = h(rng.normal(0, 0.1, N))
    g, mu, var = h(rng.uniform(0, 0.5, N)), h(rng.normal(0, 0.1, N)), h(rng.uniform(0.5, 1.5, N))
    ops = [api.constant_text("W1", W1, 12), api.constant_text("W2", W2, 12), api.constant_text("b", b, 12),
           api.constant_text("g", g, 12), api.constant_text("mu", mu, 12), api.constant_text("var", var, 12),
           api.op_text("PrunedGemm", ["x1", "x2", "W1", "W2", "b"], ["h"]), api.op_text("Dice", ["h", "g", "mu", "var"], ["y"])]
    text = api.netdef_text(ops, [("x1", 12), ("x2", 12)], [("y", 12)])
    f32 = lambda a: a.astype(np.float32)
    x1, x2 = h(rng.normal(0, 1, (m1, k1))), h(rng.normal(0, 1, (m2, k2)))
    want = orc.dice(orc.pruned_gemm(f32(x1), f32(x2), f32(W1), f32(W2), f32(b)), f32(g), f32(mu), f32(var))
    for optimize in (False, True):
        mgr = api.PredictorManager()
        mgr.load_model_text(text, optimize=optimize)
        p = mgr.create_predictor()
        keep = [p.feed("x1", x1), p.feed("x2", x2)]
        p.forward()
        got = p.output("y")
        assert got.shape == (max(m1, m2), N)
        np.testing.assert_allclose(got.astype(np.float32), want, rtol=4e-3, atol=4e-3)
        p.forward()
        assert p.launches() == (2 if optimize else 3), p.launches()      # short product + long product (+ Dice)
        p.close()
        mgr.close()


def test_binary_netdef_file(tmp_path):
    """LoadModel reads the protobuf wire format of blaze.NetDef (hand-encoded here)."""
    api = _api()

    def varint(v):
        out = bytearray()
        while True:
            b = v & 0x7f
            v >>= 7
            out.append(b | (0x80 if v else 0))
            if not v:
                return bytes(out)

    def ld(field, payload):
        return varint(field << 3 | 2) + varint(len(payload)) + payload

    def vi(field, v):
        return varint(field << 3 | 0) + varint(v)

    import struct
    shape_arg = ld(1, b"shape") + ld(6, varint(2) + varint(2))
    dtype_arg = ld(1, b"dtype") + vi(3, 1)
    value_arg = ld(1, b"value") + ld(5, struct.pack("<4f", 1.0, -2.0, 0.5, 4.0))
    const = ld(1, b"ConstantFill") + ld(4, b"x") + ld(5, shape_arg) + ld(5, dtype_arg) + ld(5, value_arg)
    sig = ld(1, b"Sigmoid") + ld(3, b"x") + ld(4, b"y")
    net = ld(1, b"bin") + ld(2, const) + ld(2, sig) + ld(5, vi(1, 1) + vi(2, 0)) + ld(7, ld(1, b"y") + vi(2, 1))
    path = tmp_path / "model.blaze"
    path.write_bytes(net)
    mgr = api.PredictorManager()
    mgr.load_model_file(str(path))
    p = mgr.create_predictor()
    p.forward()
    x = np.array([[1.0, -2.0], [0.5, 4.0]], np.float32)
    np.testing.assert_allclose(p.output("y"), 1 / (1 + np.exp(-x)), rtol=1e-6)
    p.close()
    mgr.close()


@pytest.mark.parametrize("bn_first,trans_b,dtype", [(True, False, 12), (False, False, 12), (True, True, 1), (False, False, 1)])
def test_batchnorm_folds_into_the_neighbouring_gemm(bn_first, trans_b, dtype):
    """LoadModel's optimisation pass folds a BatchNormalization with constant parameters into the Gemm it feeds
    (the shape of the reference DIN graph: bn_layer -> inner_product_layer) or follows; the folded graph is one
    kernel-library call (with the Dice behind it fused as well) and gives the un-folded graph's values."""
    api = _api()
    import orc
    rng = np.random.default_rng(7 + 2 * bn_first + trans_b)
    M, K, N = 260, 72, 80
    npdt = np.float16 if dtype == 12 else np.float32
    cast = lambda a: a.astype(npdt)
    W, b = cast(rng.normal(0, 1 / 8, (K, N))), cast(rng.normal(0, 0.1, N))
    c = K if bn_first else N
    gamma, beta = cast(rng.uniform(0.5, 1.5, c)), cast(rng.normal(0, 0.2, c))
    mean, var = cast(rng.normal(0, 0.3, c)), cast(rng.uniform(0.5, 2.0, c))
    g, mu, dv = cast(rng.uniform(0, 0.5, N)), cast(rng.normal(0, 0.1, N)), cast(rng.uniform(0.5, 1.5, N))
    consts = [api.constant_text("W", W.T if trans_b else W, dtype), api.constant_text("b", b, dtype)]
    consts += [api.constant_text(n, a, dtype) for n, a in (("gamma", gamma), ("beta", beta), ("mean", mean), ("var", var),
                                                           ("g", g), ("mu", mu), ("dv", dv))]
    gemm_args = {"transB": 1} if trans_b else None
    if bn_first:
        body = [api.op_text("BatchNormalization", ["x", "gamma", "beta", "mean", "var"], ["xn"], {"eps": 0.001}),
                api.op_text("Gemm", ["xn", "W", "b"], ["h"], gemm_args)]
    else:
        body = [api.op_text("Gemm", ["x", "W", "b"], ["h0"], gemm_args),
                api.op_text("BatchNormalization", ["h0", "gamma", "beta", "mean", "var"], ["h"], {"eps": 0.001})]
    body.append(api.op_text("Dice", ["h", "g", "mu", "dv"], ["y"]))
    text = api.netdef_text(consts + body, [("x", dtype)], [("y", dtype)])
    f32 = lambda a: a.astype(np.float32)
    x = cast(rng.normal(0, 1, (M, K)))
    if bn_first:
        h = orc.gemm_op(orc.batchnorm(f32(x), f32(gamma), f32(beta), f32(mean), f32(var), 0.001), f32(W), f32(b))
    else:
        h = orc.batchnorm(orc.gemm_op(f32(x), f32(W), f32(b)), f32(gamma), f32(beta), f32(mean), f32(var), 0.001)
    want = orc.dice(h, f32(g), f32(mu), f32(dv))
    got = {}
    for optimize in (False, True):
        mgr = api.PredictorManager()
        mgr.load_model_text(text, optimize=optimize)
        p = mgr.create_predictor()
        keep = p.feed("x", x)
        p.forward()
        p.forward()
        assert p.launches() == (1 if optimize else 3), p.launches()
        got[optimize] = p.output("y").astype(np.float32)
        p.close()
        mgr.close()
    tol = 5e-3 if dtype == 12 else 2e-4
    np.testing.assert_allclose(got[False], want, rtol=tol, atol=tol)
    np.testing.assert_allclose(got[True], want, rtol=tol, atol=tol)
