"""Second opinion on the AUGRU oracle. The reference ships no AUGRU operator or vectors (parity unpinned), so
orc_augru is a reading of the training-side TensorFlow cell; this file restates the same cell independently in
fp64 numpy, written from xdl-algorithm-solution/DIEN/script/utils.py:178-207 line by line (the _Linear layers
as explicit concatenations and matrix products), and the two must agree. A misreading of the gate order
(r | u), of the candidate input ([x, r * h]) or of the attention gating (u' = (1 - att) u,
h' = u' h + (1 - u') c) would show here."""
import numpy as np

import orc


def vec_att_gru_cell_fp64(inputs, state, att_score, gate_kernel, gate_bias, cand_kernel, cand_bias):
    """One call of VecAttGRUCell.call: inputs [B, H], state [B, H], att_score [B, 1]."""
    sigmoid = lambda z: 1.0 / (1.0 + np.exp(-z))
    # value = sigmoid(_gate_linear([inputs, state])); _Linear concatenates its arguments along axis 1
    value = sigmoid(np.concatenate([inputs, state], axis=1) @ gate_kernel + gate_bias)
    r, u = np.split(value, 2, axis=1)                       # array_ops.split(value, 2, axis=1)
    r_state = r * state
    c = np.tanh(np.concatenate([inputs, r_state], axis=1) @ cand_kernel + cand_bias)
    u = (1.0 - att_score) * u
    return u * state + (1 - u) * c


def run_fp64(x, att, Wg, bg, Wc, bc):
    B, T, H = x.shape
    h = np.zeros((B, H), np.float64)
    ys = np.empty((B, T, H), np.float64)
    for t in range(T):
        h = vec_att_gru_cell_fp64(x[:, t].astype(np.float64), h, att[:, t:t + 1].astype(np.float64),
                                  Wg.astype(np.float64), bg.astype(np.float64), Wc.astype(np.float64), bc.astype(np.float64))
        ys[:, t] = h
    return ys


def _case(seed, B, T, H):
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 0.7, (B, T, H)).astype(np.float32)
    att = rng.uniform(0, 1, (B, T)).astype(np.float32)
    Wg = rng.normal(0, 1 / np.sqrt(2 * H), (2 * H, 2 * H)).astype(np.float32)
    bg = rng.normal(1.0, 0.1, 2 * H).astype(np.float32)     # the cell initialises the gate bias to ones
    Wc = rng.normal(0, 1 / np.sqrt(2 * H), (2 * H, H)).astype(np.float32)
    bc = rng.normal(0, 0.1, H).astype(np.float32)
    return x, att, Wg, bg, Wc, bc


def test_orc_augru_agrees_with_the_fp64_restatement_of_the_tf_cell():
    for seed, (B, T, H) in enumerate([(3, 7, 4), (2, 100, 36), (5, 1, 8)]):
        args = _case(seed, B, T, H)
        got = orc.augru(*args)
        want = run_fp64(*args)
        assert np.abs(got - want).max() <= 2e-5 * max(1, T) ** 0.5, (B, T, H, np.abs(got - want).max())


def test_attention_score_one_freezes_nothing_and_zero_gives_a_plain_gru_update():
    """Properties of the gating that do not depend on either restatement's reading of the weights:
    att = 1 -> u' = 0 -> h' = c (the state is replaced by the candidate);
    att = 0 -> u' = u  -> the un-attended GRU update u h + (1 - u) c."""
    x, att, Wg, bg, Wc, bc = _case(9, 4, 6, 5)
    ones = np.ones_like(att)
    y1 = orc.augru(x, ones, Wg, bg, Wc, bc)
    H = x.shape[2]
    h = np.zeros((4, H))
    for t in range(6):
        value = 1 / (1 + np.exp(-(np.concatenate([x[:, t], h], 1) @ Wg + bg)))
        r = value[:, :H]
        h = np.tanh(np.concatenate([x[:, t], r * h], 1) @ Wc + bc)
        assert np.abs(y1[:, t] - h).max() <= 1e-5
    y0 = orc.augru(x, np.zeros_like(att), Wg, bg, Wc, bc)
    assert np.abs(y0 - run_fp64(x, np.zeros_like(att), Wg, bg, Wc, bc)).max() <= 1e-5
