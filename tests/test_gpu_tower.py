"""Fused DIN tower kernel (xb_din_tower) against the op-by-op CPU oracle: feature assembly
[user | q | his_sum | q*his_sum | att | q-his_sum], Gemm+Dice, Gemm+Dice, Gemm, Softmax."""
import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu


def _h(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def _case(R, n_cand, T, d, du, n1, n2, n3, softmax, seed):
    pkg.load()
    from x_deeplearning_b200 import ops
    rng = np.random.default_rng(seed)
    user, q = _h(rng.normal(0, 0.5, (R, du))), _h(rng.normal(0, 0.5, (R * n_cand, d)))
    k, att = _h(rng.normal(0, 0.3, (R * T, d))), _h(rng.normal(0, 0.5, (R * n_cand, d)))
    lin = lambda kk, n: (_h(rng.normal(0, 1 / np.sqrt(kk), (kk, n))), _h(rng.normal(0, 0.05, n)))
    dice = lambda n: (_h(rng.uniform(0, 0.5, n)), _h(rng.normal(0, 0.1, n)), _h(rng.uniform(0.5, 1.5, n)))
    (W1, b1), (W2, b2), (W3, b3) = lin(du + 5 * d, n1), lin(n1, n2), lin(n2, n3)
    d1, d2 = dice(n1), dice(n2)
    want = np.empty((R * n_cand, n3), np.float32)
    for r in range(R):
        rows = slice(r * n_cand, (r + 1) * n_cand)
        hs = _h(k[r * T:(r + 1) * T].sum(axis=0, dtype=np.float32, keepdims=True))       # his_sum is an fp16 tensor
        cand = np.concatenate([q[rows], np.broadcast_to(hs, (n_cand, d)), q[rows] * hs, att[rows], q[rows] - hs], 1)
        x = orc.fuse(user[r:r + 1], cand)
        y = orc.dice(orc.gemm_op(x, W1, b1), *d1)
        y = orc.dice(orc.gemm_op(y, W2, b2), *d2)
        logit = orc.gemm_op(y, W3, b3)
        want[rows] = orc.softmax(logit, axis=1) if softmax else logit
    t = torch.from_numpy
    tower = ops.DinTower(d, du, t(W1), t(b1), [t(x) for x in d1], t(W2), t(b2), [t(x) for x in d2], t(W3), t(b3),
                         softmax=softmax)
    c = lambda a: t(a).to("cuda", torch.float16)
    got = tower(c(user), c(q), c(k), c(att), R, n_cand, T)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = got.cpu().numpy()
    tol = 3e-3 if softmax else 2e-2          # probabilities; raw fp16 logits of magnitude ~1
    assert np.abs(got - want).max() <= tol, float(np.abs(got - want).max())
    if softmax:
        assert np.abs(got.sum(1) - 1).max() < 1e-5


@pytest.mark.parametrize("R,n_cand,T,d,du,n1,n2,n3,softmax", [
    (3, 200, 100, 36, 144, 200, 80, 2, True),       # the DIN tower
    (1, 1000, 100, 36, 144, 200, 80, 2, True),
    (5, 77, 7, 20, 10, 64, 32, 3, True),            # other widths, a partial tile, three classes
    (2, 130, 9, 18, 6, 48, 16, 1, False),           # d not a multiple of 4: the scalar staging path; logits
    (4, 128, 3, 8, 0, 16, 16, 8, True),             # no user columns, smallest layers, widest output
])
def test_tower_matches_oracle(R, n_cand, T, d, du, n1, n2, n3, softmax):
    _case(R, n_cand, T, d, du, n1, n2, n3, softmax, seed=R * 1000 + n_cand)


def test_tower_rejects_shapes_outside_the_kernel():
    pkg.load()
    from x_deeplearning_b200 import capi, ops
    z = lambda *s: torch.zeros(s)
    with pytest.raises(capi.XbError, match="outside the fused tower"):
        ops.DinTower(36, 144, z(324, 512), z(512), [z(512)] * 3, z(512, 80), z(80), [z(80)] * 3, z(80, 2), z(2))
