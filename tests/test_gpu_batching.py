"""Request batching through the predictor API: with InitScheduler(enable_batching = true), Forward(cb) calls
of several predictors of one model are stacked into one run (the reference's merge / run / split of
blaze/blaze/graph/hybrid_net.cc:118-176 and blaze/blaze/scheduler/batching.cc:131-191) and every predictor
gets exactly the rows it would have got running alone."""
import threading

import numpy as np
import pytest

import din_oracle
import pkg

pytestmark = pytest.mark.gpu


def _api():
    pkg.load()
    from x_deeplearning_b200 import blaze_api
    return blaze_api


@pytest.fixture
def batching():
    """Switches batching on for the predictors a test creates, and off again afterwards."""
    api = _api()

    def on(max_batch_size, timeout_micros):
        api.init_scheduler(True, max_batch_size=max_batch_size, batch_timeout_micros=timeout_micros)
    yield on
    api.init_scheduler(False)


def _din(fused_tower=True):
    from x_deeplearning_b200 import blaze_api as api, din_netdef, workloads
    model = workloads.din_model(0, item_rows=20000, cate_rows=500, user_rows=3000)
    text, _ = din_netdef.build(model, fused_tower=fused_tower)
    mgr = api.PredictorManager()
    din_netdef.register_tables(mgr, model)
    mgr.load_model_text(text, optimize=True)
    return model, mgr


def _submit_all(preds, feeds_per_pred):
    """Feeds every predictor, calls Forward(cb) on all of them, waits for the callbacks."""
    keep, done = [], [threading.Event() for _ in preds]
    for p, feeds, ev in zip(preds, feeds_per_pred, done):
        keep.append([p.feed(n, a) for n, a in feeds.items()])
        p.forward_async(ev.set)
    for ev in done:
        assert ev.wait(60), "a batched Forward never called back"
    return keep


@pytest.mark.parametrize("fused_tower", [True, False])
def test_concurrent_forwards_are_stacked_and_match_single_runs(batching, fused_tower):
    api = _api()
    from x_deeplearning_b200 import din_netdef, workloads
    batching(8, 300000)                      # a wide window: the four requests below close one batch
    model, mgr = _din(fused_tower)
    preds = [mgr.create_predictor() for _ in range(4)]
    reqs = [workloads.din_requests(model, 10 + i, requests=r, n_cand=100, seq_len=s)
            for i, (r, s) in enumerate([(1, None), (2, [100, 3]), (1, [0]), (3, None)])]
    feeds = [din_netdef.feeds_of(model, q) for q in reqs]
    # alone: the synchronous Forward() of a predictor never goes through the queue
    b0, t0 = api.batching_stats()
    singles = []
    for p, f in zip(preds, feeds):
        keep = [p.feed(n, a) for n, a in f.items()]
        p.forward()
        singles.append(p.output("output").copy())
    assert api.batching_stats() == (b0, t0)
    _submit_all(preds, feeds)
    b1, t1 = api.batching_stats()
    assert (b1 - b0, t1 - t0) == (1, 4), (b1 - b0, t1 - t0)
    for p, q, single in zip(preds, reqs, singles):
        got = p.output("output")
        assert got.shape == single.shape == (q["requests"] * q["n_cand"], 2)
        assert np.array_equal(got, single)                       # the same rows, bit for bit
        assert np.abs(got.astype(np.float32) - din_oracle.forward(model, q)).max() <= 2e-3
    for p in preds:
        p.close()
    mgr.close()


def test_requests_of_other_shapes_run_in_batches_of_their_own(batching):
    api = _api()
    from x_deeplearning_b200 import din_netdef, workloads
    batching(8, 200000)
    model, mgr = _din()
    preds = [mgr.create_predictor() for _ in range(4)]
    cands = [100, 50, 100, 50]               # candidates per user row: two kinds, interleaved
    reqs = [workloads.din_requests(model, 20 + i, requests=1 + i % 2, n_cand=c) for i, c in enumerate(cands)]
    b0, t0 = api.batching_stats()
    _submit_all(preds, [din_netdef.feeds_of(model, q) for q in reqs])
    b1, t1 = api.batching_stats()
    assert (b1 - b0, t1 - t0) == (2, 4), (b1 - b0, t1 - t0)
    for p, q in zip(preds, reqs):
        got = p.output("output").astype(np.float32)
        assert got.shape == (q["requests"] * q["n_cand"], 2)
        assert np.abs(got - din_oracle.forward(model, q)).max() <= 2e-3
    for p in preds:
        p.close()
    mgr.close()


def test_a_full_batch_closes_before_the_timeout(batching):
    api = _api()
    from x_deeplearning_b200 import din_netdef, workloads
    batching(2, 20000000)                    # 20 s window: only the size limit can close these batches in time
    model, mgr = _din()
    preds = [mgr.create_predictor() for _ in range(4)]
    reqs = [workloads.din_requests(model, 30 + i, requests=1, n_cand=64) for i in range(4)]
    b0, t0 = api.batching_stats()
    _submit_all(preds, [din_netdef.feeds_of(model, q) for q in reqs])
    b1, t1 = api.batching_stats()
    assert (b1 - b0, t1 - t0) == (2, 4), (b1 - b0, t1 - t0)
    for p, q in zip(preds, reqs):
        assert np.abs(p.output("output").astype(np.float32) - din_oracle.forward(model, q)).max() <= 2e-3
    for p in preds:
        p.close()
    mgr.close()


def test_an_operator_error_reaches_the_callback_and_output(batching):
    api = _api()
    batching(4, 1000)
    rng = np.random.default_rng(0)
    W = rng.normal(0, 0.1, (16, 8)).astype(np.float16)
    ops = [api.constant_text("W", W, 12), api.op_text("Gemm", ["x", "W"], ["y"])]
    mgr = api.PredictorManager()
    mgr.load_model_text(api.netdef_text(ops, [("x", 12)], [("y", 12)]))
    good, bad = mgr.create_predictor(), mgr.create_predictor()
    xg = rng.normal(0, 1, (5, 16)).astype(np.float16)
    xb = rng.normal(0, 1, (5, 24)).astype(np.float16)            # K does not match W: the Gemm operator refuses it
    _submit_all([good, bad], [{"x": xg}, {"x": xb}])
    want = xg.astype(np.float32) @ W.astype(np.float32)
    assert np.abs(good.output("y").astype(np.float32) - want).max() <= 2e-2
    with pytest.raises(api.BlazeError, match="batched forward failed"):
        bad.output("y")
    # the predictor stays usable
    _submit_all([bad], [{"x": xg}])
    assert np.abs(bad.output("y").astype(np.float32) - want).max() <= 2e-2
    good.close()
    bad.close()
    mgr.close()
