"""The DIN-style model on the CPU oracle, composed op by op the way the
reference graph is (blaze/tools/example_model/din/model/graph_ulf.txt): two
Embedding ops, reshape/concat to k and q, the attention unit, ReduceSum, Mul,
Concat, Fuse, then Gemm+Dice, Gemm+Dice, Gemm+Softmax."""
import numpy as np

import orc


def forward(model, req, want_parts=False):
    D = model["dims"]
    e, d, T, G = D["emb"], D["d"], D["T"], D["user_groups"]
    R, n_cand = req["requests"], req["n_cand"]
    S, A = 0, 2
    # user Embedding op: one block of G kSum items
    user_emb = np.zeros((R, G * e), np.float32)
    ones_r = np.ones(R, np.int32)
    for g in range(G):
        ids = req["user_ids"][:, g]
        orc.embedding_pool(model["user"][g], ids, np.ones(len(ids), np.float32), ones_r,
                           [dict(udf=S, out=user_emb, col=g * e)])
    # behaviour lists: kAssign trunc T, default direction kReverse, reference layout [R, T*e] per feature
    mid = np.zeros((R, T * e), np.float32)
    cat = np.zeros((R, T * e), np.float32)
    n = len(req["hist_item"])
    orc.embedding_pool(model["item"], req["hist_item"], np.ones(n, np.float32), req["seq_len"],
                       [dict(udf=A, trunc_dir=1, trunc_num=T, out=mid, col=0)])
    orc.embedding_pool(model["cate"], req["hist_cate"], np.ones(n, np.float32), req["seq_len"],
                       [dict(udf=A, trunc_dir=1, trunc_num=T, out=cat, col=0)])
    k = np.concatenate([mid.reshape(R, T, e), cat.reshape(R, T, e)], axis=2)          # reshape + concat dim 2
    # candidate Embedding op: one block item kSum | cate kSum
    q = np.zeros((R * n_cand, d), np.float32)
    ones_c = np.ones(R * n_cand, np.int32)
    nc = R * n_cand
    orc.embedding_pool(model["item"], req["cand_item"], np.ones(nc, np.float32), ones_c, [dict(udf=S, out=q, col=0)])
    orc.embedding_pool(model["cate"], req["cand_cate"], np.ones(nc, np.float32), ones_c, [dict(udf=S, out=q, col=e)])
    probs = np.empty((R * n_cand, D["tower"][2]), np.float32)
    atts = np.empty((R * n_cand, d), np.float32)
    a, tw = model["att"], model["tower"]
    w = dict(W0=a["W0"], b0=a["b0"], W1=a["W1"], b1=a["b1"], W2=a["W2"], b2=a["b2"], g0=a["g0"], m0=a["m0"],
             v0=a["v0"], g1=a["g1"], m1=a["m1"], v1=a["v1"])
    for r in range(R):
        qr = q[r * n_cand:(r + 1) * n_cand]
        # right-aligned kAssign rows: the first T - seq_len steps are zero padding and contribute nothing
        att = orc.din_attention(qr, k[r], w, act=2, seq_len=T, use_softmax=False)
        atts[r * n_cand:(r + 1) * n_cand] = att
        his_sum = k[r].sum(axis=0, dtype=np.float32, keepdims=True)                   # ReduceSum axis 1
        cand_side = np.concatenate([qr, np.broadcast_to(his_sum, qr.shape), qr * his_sum, att, qr - his_sum], 1)
        x = orc.fuse(user_emb[r:r + 1], cand_side)                                    # Fuse: user row broadcast
        y = orc.dice(orc.gemm_op(x, tw["W1"], tw["b1"]), *tw["dice1"])
        y = orc.dice(orc.gemm_op(y, tw["W2"], tw["b2"]), *tw["dice2"])
        probs[r * n_cand:(r + 1) * n_cand] = orc.softmax(orc.gemm_op(y, tw["W3"], tw["b3"]), axis=1)
    if want_parts:
        return probs, dict(user_emb=user_emb, k=k, q=q, att=atts)
    return probs
