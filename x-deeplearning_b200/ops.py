"""torch-tensor front ends of the C-ABI calls, used by tests and bench.py.

torch is plumbing here (device memory, streams); every computation is a call
into libxdlb200.so. Nothing in this file computes on the CPU or with torch ops.
"""
import ctypes as C

import torch

from . import capi
from .capi import (XB_F16, XB_F32, XB_BF16, XB_I32, XB_I64, GemmArgs, PoolGroup, TableDesc, DinAttArgs, check, lib)

_DT = {torch.float32: XB_F32, torch.float16: XB_F16, torch.bfloat16: XB_BF16, torch.int32: XB_I32,
       torch.int64: XB_I64}


def dt(t):
    return _DT[t.dtype]


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class Table:
    """An embedding table resident in HBM (xb_table_desc over torch-owned memory)."""

    def __init__(self, weights, dtype=torch.float16, keys=None, device="cuda"):
        # weights: CPU float32 [rows, dim]; keys: optional CPU int64 [rows]
        rows, dim = weights.shape
        self.rows, self.dim, self.dtype = rows, dim, dtype
        es = 2 if dtype == torch.float16 else 4
        pitch = int(lib().xb_table_row_pitch(dim, _DT[dtype]))
        self.pitch = pitch
        buf = torch.zeros((rows, pitch // es), dtype=dtype)
        buf[:, :dim] = weights.to(dtype)
        self.buf = buf.to(device)
        self.desc = TableDesc()
        self.desc.weights = self.buf.data_ptr()
        self.desc.rows, self.desc.dim, self.desc.dtype, self.desc.row_pitch_bytes = rows, dim, _DT[dtype], pitch
        self.slot_keys = self.slot_rows = None
        if keys is not None:
            slots = 16
            while slots < 2 * rows:
                slots <<= 1
            sk = torch.empty(slots, dtype=torch.int64)
            sr = torch.empty(slots, dtype=torch.int32)
            k = keys.contiguous().to(torch.int64)
            check(lib().xb_table_build_index_host(ptr(k), rows, slots, ptr(sk), ptr(sr)))
            self.slot_keys, self.slot_rows = sk.to(device), sr.to(device)
            self.desc.slot_keys, self.desc.slot_rows, self.desc.slots = (self.slot_keys.data_ptr(),
                                                                          self.slot_rows.data_ptr(), slots)


def make_group(table, ids, values, segments, items, out_dtype, segments_are_offsets=False, dim=None):
    """items: list of dict(udf, out (2-D tensor), col, trunc_dir, trunc_num, assign_stride)."""
    g = PoolGroup()
    g.table = C.pointer(table.desc) if table is not None else None
    g.ids, g.values, g.segments = ptr(ids), ptr(values), ptr(segments)
    g.n_ids = ids.numel()
    g.batch = segments.numel() - (1 if segments_are_offsets else 0)
    g.dim = table.dim if table is not None else dim
    g.id_dtype = dt(ids)
    g.segments_are_offsets = int(segments_are_offsets)
    g.out_dtype = _DT[out_dtype]
    g.n_items = len(items)
    g.values_dtype = dt(values) if values is not None else 0
    for k, it in enumerate(items):
        o = it["out"]
        assert o.dtype == out_dtype and o.dim() == 2 and o.stride(1) == 1
        g.items[k].udf = it["udf"]
        g.items[k].trunc_dir = it.get("trunc_dir", 1)
        g.items[k].trunc_num = it.get("trunc_num", 0)
        g.items[k].assign_stride = it.get("assign_stride", 0)
        g.items[k].out = o.data_ptr() + it.get("col", 0) * o.element_size()
        g.items[k].stride = o.stride(0)
    g._keep = (table, ids, values, segments, [it["out"] for it in items])
    return g


class PoolPlan:
    """A fixed set of pooling groups with its scratch buffer: one launch per 32 groups."""

    def __init__(self, groups, device="cuda"):
        self.groups = groups
        self.chunks = []
        for i in range(0, len(groups), capi.XB_MAX_POOL_GROUPS):
            part = groups[i:i + capi.XB_MAX_POOL_GROUPS]
            arr = (PoolGroup * len(part))(*part)
            need = int(lib().xb_embedding_pool_scratch_bytes(arr, len(part)))
            scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=device)
            self.chunks.append((arr, len(part), scratch, need))

    def run(self):
        s = stream()
        for arr, n, scratch, need in self.chunks:
            check(lib().xb_embedding_pool(arr, n, ptr(scratch), need, s))


def embedding_pool(groups):
    PoolPlan(groups).run()


def gemm(A, B, Y=None, bias=None, trans_a=False, trans_b=False, alpha=1.0, beta=1.0, epilogue=0, ep=(None, None, None),
         ep_count=0, nosqrt=False, engine=0, out_dtype=None, batch=1, strides=(0, 0, 0, 0), M=None, N=None, K=None,
         lda=None, ldb=None, ldy=None, bias_kind=None, stride_ep=0, ldbias=None, bias_row_group=0):
    """2-D (or explicitly strided batched) GEMM through xb_gemm. Returns Y."""
    a = GemmArgs()
    if M is None:
        M, K = (A.shape[-1], A.shape[-2]) if trans_a else (A.shape[-2], A.shape[-1])
        N = B.shape[-2] if trans_b else B.shape[-1]
    out_dtype = out_dtype or A.dtype
    if Y is None:
        Y = torch.empty((batch, M, N) if batch > 1 else (M, N), dtype=out_dtype, device=A.device)
    a.M, a.N, a.K, a.trans_a, a.trans_b, a.alpha, a.beta = M, N, K, int(trans_a), int(trans_b), alpha, beta
    a.A, a.lda, a.stride_a = A.data_ptr(), lda if lda is not None else A.stride(-2), strides[0]
    a.B, a.ldb, a.stride_b = B.data_ptr(), ldb if ldb is not None else B.stride(-2), strides[1]
    if bias is not None:
        a.bias, a.bias_dtype = bias.data_ptr(), dt(bias)
        a.bias_kind = bias_kind if bias_kind is not None else (capi.XB_BIAS_ROW if bias.dim() == 1 else capi.XB_BIAS_FULL)
        a.ldbias = ldbias if ldbias is not None else (bias.stride(-2) if bias.dim() > 1 else 0)
        a.stride_bias = strides[2]
        a.bias_row_group = bias_row_group
    a.Y, a.ldy, a.stride_y = Y.data_ptr(), ldy if ldy is not None else Y.stride(-2), strides[3]
    a.batch, a.ab_dtype, a.y_dtype = batch, dt(A), dt(Y)
    a.epilogue = epilogue
    a.ep_a, a.ep_b, a.ep_c = ptr(ep[0]), ptr(ep[1]), ptr(ep[2])
    a.ep_count, a.dice_nosqrt, a.stride_ep, a.engine = ep_count, int(nosqrt), stride_ep, engine
    check(lib().xb_gemm(C.byref(a), stream()))
    return Y


def pack_weight_kmajor(W, out_dtype=torch.float16, ldk=None, batch=1):
    """W [K,N] (or [batch,K,N]) -> [N, ldk] K-major, zero padded."""
    K, N = W.shape[-2], W.shape[-1]
    ldk = ldk or (K + 7) // 8 * 8
    out = torch.empty((batch, N, ldk) if batch > 1 else (N, ldk), dtype=out_dtype, device=W.device)
    check(lib().xb_pack_weight_kmajor(ptr(W), dt(W), K, N, W.stride(-2), ptr(out), _DT[out_dtype], ldk, batch,
                                      K * W.stride(-2) if batch > 1 else 0, N * ldk if batch > 1 else 0, stream()))
    return out


class DinAttention:
    """Weights of one attention unit packed for xb_din_attention."""

    def __init__(self, W0, b0, W1, b1, W2, b2, dice0=None, dice1=None, act=capi.XB_ACT_DICE, device="cuda"):
        # W0 [4d,h0], W1 [h0,h1], W2 [h1,1] float32 CPU tensors (Blaze layout [K,N])
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.W0 = W0.t().contiguous().to(device=device, dtype=torch.float16)
        self.W1 = W1.t().contiguous().to(device=device, dtype=torch.float16)
        self.W2 = f(W2.reshape(-1))
        self.b0, self.b1, self.b2 = f(b0), f(b1), float(b2)
        self.dice0 = [f(t) for t in dice0] if dice0 else None
        self.dice1 = [f(t) for t in dice1] if dice1 else None
        self.act = act
        self.h0, self.h1 = W0.shape[1], W1.shape[1]
        self.packed = None
        self.d = W0.shape[0] // 4

    def __call__(self, q, k, requests, n_cand, T, out=None, seq_len=None, use_softmax=False, scores=None, engine=0):
        d = q.shape[1]
        if out is None:
            out = torch.empty((requests * n_cand, d), dtype=torch.float16, device=q.device)
        a = DinAttArgs()
        a.q, a.ldq, a.k, a.ldk = q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0)
        a.seq_len, a.out, a.ldo, a.scores = ptr(seq_len), out.data_ptr(), out.stride(0), ptr(scores)
        a.requests, a.n_cand, a.T, a.d, a.h0, a.h1 = requests, n_cand, T, d, self.h0, self.h1
        a.act, a.use_softmax, a.engine = self.act, int(use_softmax), engine
        w = a.w
        w.W0, w.W1, w.W2, w.b0, w.b1, w.b2 = (self.W0.data_ptr(), self.W1.data_ptr(), self.W2.data_ptr(),
                                               self.b0.data_ptr(), self.b1.data_ptr(), self.b2)
        if self.dice0:
            w.gamma0, w.mean0, w.var0 = [t.data_ptr() for t in self.dice0]
            w.gamma1, w.mean1, w.var1 = [t.data_ptr() for t in self.dice1]
        if self.packed is None:
            # weights are constants: lay the operands out once
            n = int(lib().xb_din_attention_packed_bytes(d, self.h0, self.h1))
            self.packed = False
            if n:
                buf = torch.empty(n, dtype=torch.uint8, device=q.device)
                check(lib().xb_din_attention_pack(C.byref(a), ptr(buf), n, stream()))
                self.packed = buf
        if self.packed is not False:
            w.packed = self.packed.data_ptr()
        check(lib().xb_din_attention(C.byref(a), stream()))
        return out


def device_status():
    s = C.c_int32(0)
    check(lib().xb_device_status(C.byref(s)))
    return s.value


class DinTower:
    """Weights of the DIN tower (du+5d -> n1 -> n2 -> n3, Dice after the first two layers) packed for
    xb_din_tower. W1 [du+5d, n1], W2 [n1, n2], W3 [n2, n3] are float32 CPU tensors in Blaze's [K, N] layout."""

    def __init__(self, d, du, W1, b1, dice1, W2, b2, dice2, W3, b3, softmax=True, device="cuda"):
        h = lambda x: x.to(device=device, dtype=torch.float16).contiguous()
        f = lambda x: x.to(device=device, dtype=torch.float32).contiguous()
        self.d, self.du = d, du
        self.n1, self.n2, self.n3 = W1.shape[1], W2.shape[1], W3.shape[1]
        assert W1.shape[0] == du + 5 * d and W2.shape[0] == self.n1 and W3.shape[0] == self.n2
        self.keep = [h(W1), f(b1), f(dice1[0]), f(dice1[1]), f(dice1[2]), h(W2), f(b2), f(dice2[0]), f(dice2[1]),
                     f(dice2[2]), h(W3), f(b3)]
        self.softmax = softmax
        nbytes = lib().xb_din_tower_packed_bytes(d, self.n1, self.n2, self.n3)
        if nbytes == 0:
            raise capi.XbError("DinTower: shape outside the fused tower kernel")
        self.packed = torch.empty(nbytes, dtype=torch.uint8, device=device)
        a = self._args()
        check(lib().xb_din_tower_pack(C.byref(a), ptr(self.packed), nbytes, stream()))
        self._ws = None

    def _args(self):
        a = capi.DinTowerArgs()
        a.d, a.du, a.n1, a.n2, a.n3, a.softmax = self.d, self.du, self.n1, self.n2, self.n3, int(self.softmax)
        k = self.keep
        a.W1, a.b1, a.gamma1, a.mean1, a.var1 = k[0].data_ptr(), k[1].data_ptr(), k[2].data_ptr(), k[3].data_ptr(), k[4].data_ptr()
        a.W2, a.b2, a.gamma2, a.mean2, a.var2 = k[5].data_ptr(), k[6].data_ptr(), k[7].data_ptr(), k[8].data_ptr(), k[9].data_ptr()
        a.W3, a.b3 = k[10].data_ptr(), k[11].data_ptr()
        a.packed = self.packed.data_ptr()
        return a

    def workspace(self, requests, device="cuda"):
        """A workspace of its own for callers that keep several launches in flight on different streams."""
        return torch.empty(int(lib().xb_din_tower_workspace_bytes(requests, self.d, self.n1)), dtype=torch.uint8, device=device)

    def __call__(self, user, q, k, att, requests, n_cand, T, out=None, ws=None):
        """user [R, du], q / att [R*n_cand, d], k [R*T, d] fp16 -> probabilities [R*n_cand, n3] fp32.
        `ws`: workspace from workspace(); the default one is shared by all calls of this object (one stream)."""
        if out is None:
            out = torch.empty((requests * n_cand, self.n3), dtype=torch.float32, device=q.device)
        need = lib().xb_din_tower_workspace_bytes(requests, self.d, self.n1)
        if ws is not None:
            assert ws.numel() >= need
            a = self._args()
            a.user, a.ldu, a.q, a.ldq = user.data_ptr(), user.stride(0), q.data_ptr(), q.stride(0)
            a.k, a.ldk, a.att, a.ldatt = k.data_ptr(), k.stride(0), att.data_ptr(), att.stride(0)
            a.prob, a.requests, a.n_cand, a.T = out.data_ptr(), requests, n_cand, T
            check(lib().xb_din_tower(C.byref(a), ptr(ws), ws.numel(), stream()))
            return out
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=q.device)
        a = self._args()
        a.user, a.ldu, a.q, a.ldq = user.data_ptr(), user.stride(0), q.data_ptr(), q.stride(0)
        a.k, a.ldk, a.att, a.ldatt = k.data_ptr(), k.stride(0), att.data_ptr(), att.stride(0)
        a.prob, a.requests, a.n_cand, a.T = out.data_ptr(), requests, n_cand, T
        check(lib().xb_din_tower(C.byref(a), ptr(self._ws), self._ws.numel(), stream()))
        return out
