"""The DIEN-style model on the CPU oracle, composed op by op: Embedding ops as in the DIN graph, GRU
(blaze/blaze/operator/op/gru_op.cc:33-93), the attention MLP with sigmoid activations scoring every GRU state,
softmax over the steps, AUGRU (xdl-algorithm-solution/DIEN/script/utils.py:139-207), ReduceSum, Mul, Concat, Fuse,
Gemm+PRelu, Gemm+PRelu, Gemm+Softmax."""
import numpy as np

import din_oracle
import orc


def forward(model, req):
    D = model["dims"]
    d, T = D["d"], D["T"]
    R, n_cand = req["requests"], req["n_cand"]
    _, parts = din_oracle.forward(model, req, want_parts=True)
    user_emb, k, q = parts["user_emb"], parts["k"], parts["q"]
    g, au, tw, a = model["gru"], model["augru"], model["dien_tower"], model["att"]
    w = dict(W0=a["W0"], b0=a["b0"], W1=a["W1"], b1=a["b1"], W2=a["W2"], b2=a["b2"])
    probs = np.empty((R * n_cand, D["tower"][2]), np.float32)
    out = dict(hseq=np.empty((R, T, d), np.float32), scores=np.empty((R * n_cand, T), np.float32),
               final=np.empty((R * n_cand, d), np.float32))
    for r in range(R):
        rows = slice(r * n_cand, (r + 1) * n_cand)
        h = orc.gru(k[r], g["h2h"], g["i2h"], g["h2h_bias"], g["i2h_bias"])[0]                 # [T, d]
        _, raw = orc.din_attention(q[rows], h, w, act=1, seq_len=T, use_softmax=False, want_scores=True)
        s = orc.softmax(raw, axis=1)
        y = orc.augru(np.broadcast_to(h, (n_cand, T, d)).copy(), s, au["Wg"], au["bg"], au["Wc"], au["bc"])
        final = y[:, T - 1, :]
        his_sum = k[r].sum(axis=0, dtype=np.float32, keepdims=True)
        cand = np.concatenate([q[rows], np.broadcast_to(his_sum, (n_cand, d)), q[rows] * his_sum, final], 1)
        x = orc.fuse(user_emb[r:r + 1], cand)
        y1 = orc.prelu(orc.gemm_op(x, tw["W1"], tw["b1"]), tw["slope1"])
        y2 = orc.prelu(orc.gemm_op(y1, tw["W2"], tw["b2"]), tw["slope2"])
        probs[rows] = orc.softmax(orc.gemm_op(y2, tw["W3"], tw["b3"]), axis=1)
        out["hseq"][r], out["scores"][rows], out["final"][rows] = h, s, final
    return probs, out
