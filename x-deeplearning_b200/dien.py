"""DIEN-style model (interest extractor GRU, attention scores, AUGRU, PReLU tower) on the kernel library.

Per request r and candidate n (reference semantics: GRU = blaze/blaze/operator/op/gru_op.cc:33-93, AUGRU cell =
xdl-algorithm-solution/DIEN/script/utils.py:139-207, attention MLP and tower as in the DIN graph):
    h[r]      = GRU(k[r])                                           [T, H]
    s[n, t]   = MLP_sigmoid([q_n, h_t, q_n - h_t, q_n * h_t])       raw scores, then softmax over t
    f[n]      = last state of AUGRU(h[r], s[n])                      [H]
    prob[n]   = softmax(PReLU-MLP([user | q_n | his_sum | q_n*his_sum | f_n]))
Pooling, GRU, the fused attention unit (scores only), AUGRU and the tcgen05 GEMMs with PReLU epilogues run as
kernels of the library; the feature assembly uses the strided-copy and elementwise kernels.
"""
import ctypes as C

import numpy as np
import torch

from . import capi, ops
from .capi import check, lib
from .din import DinModel


class DienModel(DinModel):
    def __init__(self, model, device="cuda", engine=0, augru_engine=0):
        super().__init__(model, device, engine)
        self.augru_engine = augru_engine
        t = torch.from_numpy
        h = lambda x: t(np.ascontiguousarray(x)).to(device=device, dtype=torch.float16)
        f32 = lambda x: t(np.ascontiguousarray(x)).to(device=device, dtype=torch.float32)
        a = model["att"]
        # the same MLP weights as the DIN unit, sigmoid activations (no Dice parameters)
        self.att_sig = ops.DinAttention(t(a["W0"]), t(a["b0"]), t(a["W1"]), t(a["b1"]), t(a["W2"]), float(a["b2"][0]),
                                        act=capi.XB_ACT_SIGMOID, device=device)
        self.gru = {k: h(v) for k, v in model["gru"].items()}
        self.augru = {k: h(v) for k, v in model["augru"].items()}
        tw = model["dien_tower"]
        D = self.D
        self.dtin = D["user_groups"] * D["emb"] + 4 * D["d"]
        # the tower input is assembled by xb_din_tower_input, which writes a fifth candidate-side segment
        # (q - his_sum) after the four this model uses: the first layer's packed weight is zero there
        self.dldx = (D["user_groups"] * D["emb"] + 5 * D["d"] + 7) // 8 * 8
        self.dW1 = ops.pack_weight_kmajor(t(tw["W1"]).to(device), torch.float16, ldk=self.dldx)
        self.dW2 = ops.pack_weight_kmajor(t(tw["W2"]).to(device), torch.float16)
        self.dW3 = ops.pack_weight_kmajor(t(tw["W3"]).to(device), torch.float16)
        self.db = [f32(tw["b1"]), f32(tw["b2"]), f32(tw["b3"])]
        self.dslope = [f32(tw["slope1"]), f32(tw["slope2"])]

    def forward_dien(self, p):
        """Inputs already uploaded by DinModel.upload(). Returns probabilities [R*n_cand, 2] fp32."""
        D, dev, L, s = self.D, self.dev, lib(), ops.stream()
        R, n_cand, T, H = p["R"], p["n_cand"], D["T"], D["d"]
        du, N = D["user_groups"] * D["emb"], R * n_cand
        F16, F32 = capi.XB_F16, capi.XB_F32
        e16 = lambda *sh: torch.empty(sh, dtype=torch.float16, device=dev)
        p["pool"].run()
        k, q = p["k"], p["q"]                                      # [R, T*H], [N, H]
        # interest extractor
        hseq = e16(R, T * H)
        g = self.gru
        check(L.xb_gru(ops.ptr(k), ops.ptr(hseq), R, T, H, ops.ptr(g["i2h"]), ops.ptr(g["h2h"]), ops.ptr(g["i2h_bias"]),
                       ops.ptr(g["h2h_bias"]), F16, s))
        # attention scores of every GRU state against the candidate, softmax over the steps
        raw = torch.empty((N, T), dtype=torch.float32, device=dev)
        self.att_sig(q, hseq.view(R * T, H), R, n_cand, T, out=p["att"], scores=raw)
        sm = torch.empty_like(raw)
        check(L.xb_softmax(ops.ptr(raw), ops.ptr(sm), N, T, 1, F32, s))
        score16 = e16(N, T)
        check(L.xb_copy2d(ops.ptr(sm), T, F32, ops.ptr(score16), T, F16, N, T, s))
        # interest evolution: every candidate runs the AUGRU over its request's GRU states, which are read once
        # per 128-candidate tile; only the final state is kept
        final = e16(N, H)
        a = self.augru
        check(L.xb_augru_shared(ops.ptr(hseq), ops.ptr(score16), ops.ptr(final), R, n_cand, T, H, ops.ptr(a["Wg"]),
                                ops.ptr(a["bg"]), ops.ptr(a["Wc"]), ops.ptr(a["bc"]), self.augru_engine, s))
        # tower input [user | q | his_sum | q*his_sum | final state | (q - his_sum: zero weights)]
        X = e16(N, self.dldx)
        check(L.xb_din_tower_input(ops.ptr(p["user_emb"]), du, ops.ptr(q), H, ops.ptr(k), H, ops.ptr(final), H, ops.ptr(X),
                                   self.dldx, R, n_cand, T, H, du, s))
        E = capi
        t1, t2, t3 = D["tower"]
        y1, y2 = e16(N, t1), e16(N, t2)
        logit = torch.empty((N, t3), dtype=torch.float32, device=dev)
        ops.gemm(X, self.dW1, Y=y1, bias=self.db[0], trans_b=True, epilogue=E.XB_EPI_PRELU, ep=(self.dslope[0], None, None),
                 ep_count=t1, engine=self.engine, K=self.dldx, M=N, N=t1)
        ops.gemm(y1, self.dW2, Y=y2, bias=self.db[1], trans_b=True, epilogue=E.XB_EPI_PRELU, ep=(self.dslope[1], None, None),
                 ep_count=t2, engine=self.engine, K=t1, M=N, N=t2)
        ops.gemm(y2, self.dW3, Y=logit, bias=self.db[2], trans_b=True, engine=self.engine, K=t2, M=N, N=t3)
        prob = torch.empty_like(logit)
        check(L.xb_softmax(ops.ptr(logit), ops.ptr(prob), N, t3, 1, F32, s))
        keep = (hseq, raw, sm, score16, X, final, y1, y2, logit)                       # alive until the stream drains
        p["dien_keep"] = keep
        return prob, dict(hseq=hseq, scores=sm, final=final)
