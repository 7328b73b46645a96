"""Whole DIN-style model: GPU pipeline vs the op-by-op CPU oracle, final probabilities within 2e-3."""
import numpy as np
import pytest
import torch

import din_oracle
import pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("emb_sigma,seq", [(0.01, None), (0.5, None), (0.5, [100, 3, 0])])
def test_din_probabilities_match_oracle(emb_sigma, seq):
    pkg.load()
    from x_deeplearning_b200 import din, ops, workloads
    model = workloads.din_model(0, item_rows=20000, cate_rows=500, user_rows=3000, emb_sigma=emb_sigma)
    R = 3
    req = workloads.din_requests(model, 1, requests=R, n_cand=200, seq_len=seq)
    want, parts = din_oracle.forward(model, req, want_parts=True)
    net = din.DinModel(model)
    staged = net.stage(req)
    p = net.upload(staged)
    prob = net.forward_device(p)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    # pooled embeddings: bit-exact gathers (fp16 rows, one id per segment)
    np.testing.assert_array_equal(p["q"].float().cpu().numpy(), parts["q"])
    np.testing.assert_array_equal(p["k"].float().cpu().numpy().reshape(R, 100, 36), parts["k"])
    np.testing.assert_array_equal(p["user_emb"].float().cpu().numpy(), parts["user_emb"])
    got = prob.cpu().numpy()
    assert np.abs(got - want).max() <= 2e-3, np.abs(got - want).max()
    assert np.abs(got.sum(1) - 1).max() < 1e-5
    # the first tower layer as one Gemm over the full concat (no pruned product) stays within the same bound
    for pruned in (False, True):
        got_ops = net.forward_device(p, pruned=pruned, fused_tower=False).cpu().numpy()
        assert np.abs(got_ops - want).max() <= 2e-3, (pruned, np.abs(got_ops - want).max())
    prob = net.forward_device(p)
    # end to end from pinned host buffers gives the same answer
    got2 = net.forward(staged).numpy()
    np.testing.assert_array_equal(got, got2)


def test_din_at_the_benchmark_size_matches_oracle():
    """The configuration the benchmark times: 5 M x 18 item table, 10 k categories, 8 x 100 k user groups,
    one request of 1 user x 1000 candidates, T = 100."""
    pkg.load()
    from x_deeplearning_b200 import din, ops, workloads
    model = workloads.din_model(seed=0)
    assert model["item"].shape[0] == 5_000_000
    req = workloads.din_requests(model, 17, requests=1, n_cand=1000)
    want, parts = din_oracle.forward(model, req, want_parts=True)
    net = din.DinModel(model)
    p = net.upload(net.stage(req))
    got = net.forward_device(p).cpu().numpy()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    np.testing.assert_array_equal(p["q"].float().cpu().numpy(), parts["q"])
    assert got.shape == (1000, 2)
    assert np.abs(got - want).max() <= 2e-3, np.abs(got - want).max()
