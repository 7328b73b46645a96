"""DIEN-style model (GRU -> attention scores -> AUGRU -> PReLU tower): GPU pipeline against the op-by-op CPU
oracle. The AUGRU cell has no counterpart in the reference's inference code, so this parity is against the
restated training-side cell only."""
import numpy as np
import pytest
import torch

import dien_oracle
import pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("augru_engine", [1, 0])        # CUDA-core AUGRU, then the tcgen05 one (XB_GEMM_AUTO picks it)
@pytest.mark.parametrize("R,n_cand,emb_sigma", [(2, 64, 0.5), (1, 1000, 0.3)])
def test_dien_probabilities_match_oracle(R, n_cand, emb_sigma, augru_engine):
    pkg.load()
    from x_deeplearning_b200 import dien, ops, workloads
    model = workloads.dien_model(0, item_rows=20000, cate_rows=500, user_rows=3000, emb_sigma=emb_sigma)
    req = workloads.din_requests(model, 5, requests=R, n_cand=n_cand)
    want, wparts = dien_oracle.forward(model, req)
    net = dien.DienModel(model, augru_engine=augru_engine)
    p = net.upload(net.stage(req))
    prob, parts = net.forward_dien(p)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    f = lambda t: t.float().cpu().numpy()
    T, H = 100, 36
    np.testing.assert_allclose(f(parts["hseq"]).reshape(R, T, H), wparts["hseq"], rtol=0, atol=4e-3)      # fp16 GRU states
    np.testing.assert_allclose(f(parts["scores"]), wparts["scores"], rtol=0, atol=2e-3)                 # softmax over steps
    np.testing.assert_allclose(f(parts["final"]), wparts["final"], rtol=0, atol=8e-3)                   # fp16 AUGRU state
    got = f(prob)
    assert np.abs(got - want).max() <= 4e-3, np.abs(got - want).max()
    assert np.abs(got.sum(1) - 1).max() < 1e-5
