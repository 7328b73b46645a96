"""The DIN-style model end to end through the host runtime's Predictor API (host buffers in,
probabilities out) against the op-by-op CPU oracle: final probabilities within 2e-3."""
import numpy as np
import pytest
import torch

import din_oracle
import pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused_tower", [True, False])
@pytest.mark.parametrize("emb_sigma,seq", [(0.5, None), (0.5, [100, 17, 0]), (0.01, None)])
def test_predictor_din_matches_oracle(emb_sigma, seq, fused_tower):
    pkg.load()
    from x_deeplearning_b200 import blaze_api as api, din_netdef, workloads
    model = workloads.din_model(0, item_rows=20000, cate_rows=500, user_rows=3000, emb_sigma=emb_sigma)
    req = workloads.din_requests(model, 2, requests=3, n_cand=200, seq_len=seq)
    want = din_oracle.forward(model, req)
    text, feed_names = din_netdef.build(model, fused_tower=fused_tower)
    mgr = api.PredictorManager()
    din_netdef.register_tables(mgr, model)
    mgr.load_model_text(text, optimize=True)
    p = mgr.create_predictor(device_type=1, device_id=0)
    assert p.names("input") == feed_names and p.names("output") == ["output"]
    feeds = din_netdef.feeds_of(model, req)
    keep = [p.feed(n, a) for n, a in feeds.items()]
    p.forward()
    got = p.output("output").astype(np.float32)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 2e-3, np.abs(got - want).max()
    # a second request batch of another size re-uses the predictor
    req2 = workloads.din_requests(model, 3, requests=1, n_cand=77)
    keep = [p.feed(n, a) for n, a in din_netdef.feeds_of(model, req2).items()]
    p.forward()
    got2 = p.output("output").astype(np.float32)
    assert np.abs(got2 - din_oracle.forward(model, req2)).max() <= 2e-3
    # pooling (scan + pool) x2, 2 concat copies, attention, then the two tower kernels or, op by op,
    # tower input, pruned product (2 launches), 2 gemm, softmax
    assert p.launches() == (9 if fused_tower else 13), p.launches()
    p.close()
    mgr.close()


def test_qed_file_written_by_the_reference_store_loads_into_hbm(tmp_path):
    """A QED file produced by the reference's own store code is read by the b200 puller."""
    import orc
    if orc.ref_lib() is None:
        pytest.skip("oracle/_ref not built")
    pkg.load()
    from x_deeplearning_b200 import blaze_api as api
    rng = np.random.default_rng(5)
    keys = rng.choice(1 << 40, size=300, replace=False).astype(np.int64)
    w = rng.normal(0, 1, (300, 6)).astype(np.float32)
    path = str(tmp_path / "t.qed")
    st = orc.RefStore({"104_7": (keys, w), "other": (keys[:5], w[:5, :4].copy())}, path)
    counts = np.array([3, 0, 2, 4], np.int32)
    ids = keys[rng.integers(0, 300, counts.sum())]
    ids[1] = 12345                                            # not in the table
    vals = rng.normal(1, 0.3, len(ids)).astype(np.float32)
    want = np.zeros((4, 6 + 12), np.float32)
    items = [dict(udf=0, out=want, col=0), dict(udf=2, trunc_dir=0, trunc_num=2, out=want, col=6)]
    assert st.get("104_7", ids, vals, counts, items) == 0
    st.close()
    conf = ('feature_group_config { feature_group: "f" table_name: "104_7" dim: 6 }\n'
            'block_config { embedding_block_config_item { feature_group: "f" udf_type: 0 }\n'
            ' embedding_block_config_item { feature_group: "f" udf_type: 2 trunc_direction: kInorder trunc_num: 2 } }\n')
    # one feature group feeding two items of one block
    text = api.netdef_text([api.op_text("Embedding", ["f.ids", "f.values", "f.segments"], ["out"], {"embedding_config": conf})],
                           [("f.ids", 10), ("f.values", 1), ("f.segments", 2)], [("out", 1)])
    mgr = api.PredictorManager()
    mgr.load_sparse(path, "qed_sparse_puller")
    mgr.load_model_text(text)
    p = mgr.create_predictor()
    keep = [p.feed("f.ids", ids), p.feed("f.values", vals), p.feed("f.segments", counts)]
    p.forward()
    np.testing.assert_allclose(p.output("out"), want, rtol=1e-6, atol=1e-6)
    p.close()
    mgr.close()


def test_one_manager_serves_predictors_on_two_devices():
    """One process, one PredictorManager, CreatePredictor(type, device_id) for two device ids (the reference's
    deployment model, blaze/blaze/api/cpp_api/predictor_manager_impl.cc:142-177): tables are replicated per
    device, launch attributes are set per device, and both predictors match the oracle."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible devices")
    pkg.load()
    from x_deeplearning_b200 import blaze_api as api, din_netdef, workloads
    model = workloads.din_model(0, item_rows=20000, cate_rows=500, user_rows=3000, emb_sigma=0.5)
    text, _ = din_netdef.build(model)
    mgr = api.PredictorManager()
    din_netdef.register_tables(mgr, model)
    mgr.load_model_text(text, optimize=True)
    preds = [mgr.create_predictor(device_type=1, device_id=d) for d in (0, 1)]
    for seed, p in zip((5, 6), preds):
        req = workloads.din_requests(model, seed, requests=2, n_cand=300)
        keep = [p.feed(n, a) for n, a in din_netdef.feeds_of(model, req).items()]
        p.forward()
        got = p.output("output").astype(np.float32)
        assert np.abs(got - din_oracle.forward(model, req)).max() <= 2e-3
    # and again in the other order: both devices keep working side by side
    for seed, p in zip((8, 7), preds[::-1]):
        req = workloads.din_requests(model, seed, requests=1, n_cand=130)
        keep = [p.feed(n, a) for n, a in din_netdef.feeds_of(model, req).items()]
        p.forward()
        assert np.abs(p.output("output").astype(np.float32) - din_oracle.forward(model, req)).max() <= 2e-3
    for p in preds:
        p.close()
    mgr.close()
    torch.cuda.set_device(0)


@pytest.mark.parametrize("optimize", [True, False])
def test_unfused_graph_through_the_predictor(optimize):
    """The op-by-op graph of one request (what the reference's own CPU operators run in the benchmark's reference
    arm), fp16, on the GPU: op by op as written, and rewritten by the fusion pass into DinAttention + DinTower."""
    pkg.load()
    from x_deeplearning_b200 import blaze_api as api, din_netdef, workloads
    model = workloads.din_model(0, item_rows=20000, cate_rows=500, user_rows=3000, emb_sigma=0.5)
    text, _ = din_netdef.build_unfused(model, dtype=12, device_type=1)
    mgr = api.PredictorManager()
    din_netdef.register_tables(mgr, model)
    mgr.load_model_text(text, optimize=optimize)
    assert ("DinTower" in mgr.op_types()) == optimize
    p = mgr.create_predictor(device_type=1, device_id=0)
    launches = []
    for seed, n_cand, seq in ((4, 200, None), (5, 77, [31])):
        req = workloads.din_requests(model, seed, requests=1, n_cand=n_cand, seq_len=seq)
        keep = [p.feed(n, a) for n, a in din_netdef.feeds_of(model, req).items()]
        p.forward()
        got = p.output("output").astype(np.float32)
        want = din_oracle.forward(model, req)
        assert got.shape == want.shape
        assert np.abs(got - want).max() <= 2e-3, np.abs(got - want).max()
        launches.append(p.launches())
    # (the first run also packs the weights; the second one is the steady state)
    assert (launches[1] <= 12) if optimize else (launches[1] >= 25), launches
    p.close()
    mgr.close()
