"""Fused DIN attention unit: both engines against the op-by-op CPU oracle."""
import numpy as np
import pytest
import torch

import orc
import pkg

pytestmark = pytest.mark.gpu


def _weights(rng, d, h0, h1):
    r16 = lambda a: np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
    w = dict(W0=r16(rng.normal(0, 1 / np.sqrt(4 * d), (4 * d, h0))), b0=r16(rng.normal(0, 0.1, h0)),
             W1=r16(rng.normal(0, 1 / np.sqrt(h0), (h0, h1))), b1=r16(rng.normal(0, 0.1, h1)),
             W2=r16(rng.normal(0, 1 / np.sqrt(h1), (h1, 1))), b2=r16(rng.normal(0, 0.1, 1)))
    for i, h in ((0, h0), (1, h1)):
        w["g%d" % i] = r16(rng.uniform(0, 0.5, h))
        w["m%d" % i] = r16(rng.normal(0, 0.1, h))
        w["v%d" % i] = r16(rng.uniform(0.5, 1.5, h))
    return w


def _case(engine_name, R, n_cand, T, d, h0, h1, act, softmax, seq_lens=None, seed=0, sigma=0.5):
    pkg.load()
    from x_deeplearning_b200 import ops, capi
    engine = {"simt": capi.XB_GEMM_SIMT, "tc": capi.XB_GEMM_TCGEN05, "pair": capi.XB_ATT_ENGINE_PAIR,
              "split": capi.XB_ATT_ENGINE_SPLIT}[engine_name]
    rng = np.random.default_rng(seed)
    w = _weights(rng, d, h0, h1)
    q = rng.normal(0, sigma, (R * n_cand, d)).astype(np.float16)
    k = rng.normal(0, sigma, (R * T, d)).astype(np.float16)
    t = torch.from_numpy
    att = ops.DinAttention(t(w["W0"]), t(w["b0"]), t(w["W1"]), t(w["b1"]), t(w["W2"]), float(w["b2"][0]),
                           dice0=[t(w["g0"]), t(w["m0"]), t(w["v0"])], dice1=[t(w["g1"]), t(w["m1"]), t(w["v1"])],
                           act=act)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device="cuda") if seq_lens is not None else None
    want_scores = not (softmax and engine_name in ("tc", "pair", "split"))
    scores = torch.zeros((R * n_cand, T), device="cuda") if want_scores else None
    out = att(t(q).cuda(), t(k).cuda(), R, n_cand, T, seq_len=sl, use_softmax=softmax, scores=scores, engine=engine)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = out.float().cpu().numpy()
    for r in range(R):
        L = T if seq_lens is None else seq_lens[r]
        o, s = orc.din_attention(q[r * n_cand:(r + 1) * n_cand].astype(np.float32), k[r * T:(r + 1) * T].astype(np.float32),
                                 w, act=act, seq_len=L, use_softmax=softmax, want_scores=True)
        if want_scores:
            gs = scores[r * n_cand:(r + 1) * n_cand].cpu().numpy()
            assert np.abs(gs - s).max() <= (5e-3 if engine_name in ("tc", "pair", "split") else 1e-3), np.abs(gs - s).max()
        g = got[r * n_cand:(r + 1) * n_cand]
        bound = (np.abs(s) @ np.abs(k[r * T:(r + 1) * T].astype(np.float32)))
        assert (np.abs(g - o) <= 4e-3 * (1 + bound)).all(), float(np.abs(g - o).max())


@pytest.mark.parametrize("engine", ["simt", "tc", "pair", "split"])
def test_din_shape_dice_no_softmax(engine):
    _case(engine, R=2, n_cand=300, T=100, d=36, h0=80, h1=40, act=2, softmax=False)


@pytest.mark.parametrize("engine", ["simt", "tc", "pair", "split"])
def test_shipped_graph_variant_sigmoid_masked_softmax(engine):
    _case(engine, R=3, n_cand=130, T=100, d=36, h0=80, h1=40, act=1, softmax=True, seq_lens=[100, 37, 1], seed=1)


@pytest.mark.parametrize("engine", ["simt", "tc", "pair", "split"])
def test_ragged_and_empty_sequences(engine):
    _case(engine, R=4, n_cand=70, T=20, d=36, h0=80, h1=40, act=2, softmax=False, seq_lens=[20, 0, 1, 7], seed=2)


@pytest.mark.parametrize("engine", ["simt", "tc", "pair", "split"])
def test_other_dims(engine):
    _case(engine, R=1, n_cand=129, T=33, d=16, h0=32, h1=16, act=0, softmax=False, seed=3)
    if engine != "split":                  # the split engine does not take behaviour lists this short
        _case(engine, R=1, n_cand=5, T=3, d=20, h0=48, h1=24, act=2, softmax=False, seed=4)
    _case(engine, R=2, n_cand=140, T=11, d=18, h0=32, h1=16, act=1, softmax=False, seed=5)    # d not a multiple of 4


def test_per_step_engine_with_two_layer2_operand_buffers():
    """A first hidden layer of 96 leaves tensor memory for two (not three) layer-2 operand buffers: the
    layer-1 warps then wait for the layer-2 MMA two steps back before they overwrite its operand."""
    _case("tc", R=2, n_cand=200, T=37, d=36, h0=96, h1=32, act=2, softmax=False, seq_lens=[37, 12], seed=6)
    _case("tc", R=1, n_cand=128, T=2, d=32, h0=96, h1=48, act=1, softmax=True, seed=7)


def test_split_engine_walks_several_requests_and_tiles_per_cta():
    """More tiles than SMs: every CTA of the persistent engine walks a run of tiles that crosses request
    boundaries (ragged sequence lengths, a partial last tile per request, an empty sequence in the middle)."""
    _case("split", R=40, n_cand=1000, T=100, d=36, h0=80, h1=40, act=2, softmax=False,
          seq_lens=[100, 99, 0, 1, 2, 3, 50, 100] * 5, seed=6)


def test_split_engine_declines_very_short_lists():
    pkg.load()
    from x_deeplearning_b200 import capi
    with pytest.raises(capi.XbError, match="outside the split engine"):
        _case("split", R=1, n_cand=5, T=3, d=20, h0=48, h1=24, act=2, softmax=False, seed=4)
