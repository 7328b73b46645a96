"""The reference's own dense CPU operators (oracle/_ref/libblaze_cpu.so, compiled unmodified from a reference
checkout) against (1) the expected values its own golden nets carry and (2) the plain-C oracle on random shapes of
the DIN-style model's size. Skipped where the library was not built."""
import json
import os

import numpy as np
import pytest

import orc
import pkg
import refnet

HERE = os.path.dirname(os.path.abspath(__file__))
FIX = json.load(open(os.path.join(HERE, "golden", "blaze_op_fixtures.json")))
needs_ref = pytest.mark.skipif(refnet.lib() is None, reason="oracle/_ref/libblaze_cpu.so not built")


def _api():
    pkg.load()
    from x_deeplearning_b200 import blaze_api
    return blaze_api


@needs_ref
@pytest.mark.parametrize("name", sorted(n for n in FIX if "embedding" not in n))
def test_reference_library_reproduces_its_own_golden_nets(name):
    api = _api()
    net = FIX[name]
    r = refnet.RefNet(api.fixture_to_text(net, device_type=0))
    r.run()
    for out, exp in net["expected"].items():
        want = np.array([float(str(v).rstrip("f")) for v in exp["values"]], np.float64).reshape(exp["shape"])
        got = r.output(out)
        assert list(got.shape) == list(exp["shape"])
        np.testing.assert_allclose(got.astype(np.float64), want, rtol=0, atol=1e-6)
    r.close()


@needs_ref
def test_oracle_matches_the_reference_operators_on_din_sized_shapes():
    """Gemm + bias, Dice, PRelu, Sigmoid, Softmax, FusedParallelGemm at the sizes of the attention unit and the
    tower (the golden nets only hold tiny shapes)."""
    api = _api()
    rng = np.random.default_rng(3)
    M, K, N = 1000, 144, 80
    x = rng.normal(0, 0.5, (M, K)).astype(np.float32)
    W = rng.normal(0, 1 / 12, (K, N)).astype(np.float32)
    b = rng.normal(0, 0.1, N).astype(np.float32)
    g, mu, var = (rng.uniform(0, 0.5, N).astype(np.float32), rng.normal(0, 0.1, N).astype(np.float32),
                  rng.uniform(0.5, 1.5, N).astype(np.float32))
    slope = rng.uniform(0.1, 0.4, N).astype(np.float32)
    ops = [api.constant_text("W", W, 1), api.constant_text("b", b, 1), api.constant_text("g", g, 1),
           api.constant_text("mu", mu, 1), api.constant_text("var", var, 1), api.constant_text("slope", slope, 1),
           api.op_text("Gemm", ["x", "W", "b"], ["h"]), api.op_text("Dice", ["h", "g", "mu", "var"], ["dice"]),
           api.op_text("PRelu", ["h", "slope"], ["prelu"]), api.op_text("Sigmoid", ["h"], ["sig"]),
           api.op_text("Softmax", ["h"], ["soft"], {"axis": 1})]
    outs = ["dice", "prelu", "sig", "soft"]          # (a blob other operators consume is not an external output)
    r = refnet.RefNet(api.netdef_text(ops, [("x", 1)], [(o, 1) for o in outs], device_type=0))
    r.feed("x", x)
    r.run()
    h = orc.gemm_op(x, W, b)
    want = {"dice": orc.dice(h, g, mu, var), "prelu": orc.prelu(h, slope), "sig": orc.sigmoid(h),
            "soft": orc.softmax(h, axis=1)}
    for o in outs:
        # the BLAS may add in another order than the oracle's k-ascending loop: fp32 re-association only
        np.testing.assert_allclose(r.output(o), want[o], rtol=2e-5, atol=2e-5, err_msg=o)
    r.close()


@needs_ref
def test_reference_library_names_its_blas():
    assert "OpenBLAS" in refnet.blas_name() or "naive" in refnet.blas_name()


def _din_qed(model, path):
    tables = {"item": (np.arange(len(model["item"]), dtype=np.int64), model["item"]),
              "cate": (np.arange(len(model["cate"]), dtype=np.int64), model["cate"])}
    for g, w in enumerate(model["user"]):
        tables["user%d" % g] = (np.arange(len(w), dtype=np.int64), w)
    orc.RefStore(tables, path).close()


@needs_ref
def test_unfused_din_graph_on_the_reference_operators_matches_the_oracle_composition(tmp_path):
    """The whole DIN-style model, one request, op by op on the reference's own CPU operators (Embedding served by
    its qed_sparse_puller from a QED file its own store code wrote) against the oracle's composition."""
    if orc.ref_lib() is None:
        pytest.skip("oracle/_ref/libqed_ref.so not built")
    pkg.load()
    from x_deeplearning_b200 import din_netdef, workloads
    import din_oracle
    model = workloads.din_model(0, item_rows=3000, cate_rows=200, user_rows=500, emb_sigma=0.5)
    path = str(tmp_path / "din.qed")
    _din_qed(model, path)
    text, _ = din_netdef.build_unfused(model)
    net = refnet.RefNet(text, path)
    for seed, n_cand, seq in ((1, 60, None), (2, 17, [33])):
        req = workloads.din_requests(model, seed, requests=1, n_cand=n_cand, seq_len=seq)
        for n, a in din_netdef.feeds_of(model, req).items():
            net.feed(n, a.astype(np.float32) if n.endswith(".values") else a)
        net.run()
        got = net.output("output")
        want = din_oracle.forward(model, req)
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= 2e-5, np.abs(got - want).max()
    net.close()
