"""ctypes access to the CPU checkers (oracle/liboracle.so and, when built,
oracle/_ref/libqed_ref.so). Test infrastructure: imported by tests/, by
bench.py's CPU-baseline legs and by __graft_entry__.smoke() only."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

_f = C.POINTER(C.c_float)
_i64 = C.POINTER(C.c_int64)
_i32 = C.POINTER(C.c_int32)


def _p(a, t):
    return a.ctypes.data_as(t) if a is not None else None


def reference_root():
    """Root of a reference checkout when one is mounted (XDL_REFERENCE, or the sibling `reference` folder of
    the repository), else ""."""
    cands = [os.environ.get("XDL_REFERENCE", ""),
             os.path.join(os.path.dirname(os.path.dirname(ORACLE_DIR)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "blaze", "blaze", "store")):
            return c
    return ""


def build(openmp=False):
    subprocess.check_call(["make", "-s", "-C", ORACLE_DIR, "oracle"])
    ref = reference_root()
    if ref:
        subprocess.call(["make", "-s", "-C", ORACLE_DIR, "ref", "REF=" + ref], stdout=subprocess.DEVNULL)


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(ORACLE_DIR, "liboracle.so")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(
                os.path.join(ORACLE_DIR, "oracle.c")):
            build()
        _lib = C.CDLL(path)
        _lib.orc_index_create.restype = C.c_void_p
        _lib.orc_index_create.argtypes = [_i64, C.c_int64]
        _lib.orc_index_destroy.argtypes = [C.c_void_p]
    return _lib


class AttW(C.Structure):
    _fields_ = [(n, _f) for n in ("W0", "b0", "W1", "b1", "W2", "b2", "g0", "m0", "v0", "g1", "m1", "v1")]


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def embedding_pool(table, keys, values, key_num, items, table_keys=None):
    """items: list of dict(udf, trunc_dir, trunc_num, out (2-D fp32 array view base),
    col (column offset), assign_stride). Writes into the given out arrays."""
    L = lib()
    table = f32(table)
    rows, dim = table.shape
    keys = np.ascontiguousarray(keys, dtype=np.int64)
    values = f32(values)
    key_num = np.ascontiguousarray(key_num, dtype=np.int32)
    n = len(items)
    udf = (C.c_int * n)(*[it["udf"] for it in items])
    td = (C.c_int * n)(*[it.get("trunc_dir", 1) for it in items])
    tn = (C.c_int * n)(*[it.get("trunc_num", 0) for it in items])
    ast = (C.c_int * n)(*[it.get("assign_stride", dim) for it in items])
    outs = (_f * n)()
    strides = (C.c_int64 * n)()
    for k, it in enumerate(items):
        o = it["out"]
        assert o.dtype == np.float32 and o.flags["C_CONTIGUOUS"] and o.ndim == 2
        outs[k] = C.cast(o.ctypes.data + 4 * it.get("col", 0), _f)
        strides[k] = o.shape[1]
    ix = None
    if table_keys is not None:
        tk = np.ascontiguousarray(table_keys, dtype=np.int64)
        ix = L.orc_index_create(_p(tk, _i64), len(tk))
    L.orc_embedding_pool(_p(table, _f), C.c_int64(rows), dim, C.c_void_p(ix), _p(keys, _i64),
                         _p(values, _f), _p(key_num, _i32), C.c_int64(len(key_num)), n, udf, td, tn,
                         ast, outs, strides)
    if ix:
        L.orc_index_destroy(C.c_void_p(ix))


def gemm_op(A, B, bias=None, transa=False, transb=False, alpha=1.0, beta=1.0):
    A, B = f32(A), f32(B)
    M, K = (A.shape[1], A.shape[0]) if transa else A.shape
    N = B.shape[0] if transb else B.shape[1]
    Y = np.empty((M, N), np.float32)
    brow = 1
    if bias is not None:
        bias = f32(bias)
        brow = 1 if bias.ndim == 1 else M
    lib().orc_gemm_op(int(transa), int(transb), C.c_int64(M), C.c_int64(N), C.c_int64(K),
                      C.c_float(alpha), _p(A, _f), _p(B, _f), C.c_float(beta), _p(bias, _f),
                      C.c_int64(brow), _p(Y, _f))
    return Y


def pruned_gemm(x1, x2, w1, w2, bias=None, alpha=1.0, beta=1.0):
    """PrunedGemm with the shorter of x1 / x2 broadcast over row groups of the longer one."""
    x1, x2, w1, w2 = f32(x1), f32(x2), f32(w1), f32(w2)
    if x1.shape[0] <= x2.shape[0]:
        xs, ws, xl, wl = x1, w1, x2, w2
    else:
        xs, ws, xl, wl = x2, w2, x1, w1
    M, N = xl.shape[0], wl.shape[1]
    assert M % xs.shape[0] == 0
    Y = np.empty((M, N), np.float32)
    if bias is not None:
        bias = f32(bias).ravel()
    lib().orc_pruned_gemm(C.c_int64(M), C.c_int64(N), C.c_int64(M // xs.shape[0]), C.c_int64(xs.shape[1]),
                          C.c_int64(xl.shape[1]), C.c_float(alpha), C.c_float(beta), _p(xs, _f), _p(ws, _f),
                          _p(xl, _f), _p(wl, _f), _p(bias, _f), _p(Y, _f))
    return Y


def gemm_strided_batched(A, sa, B, sb, M, N, K, batch, transa=False, transb=False, alpha=1.0):
    A, B = f32(A).ravel(), f32(B).ravel()
    Cm = np.zeros((batch, M, N), np.float32)
    lib().orc_gemm_strided_batched(int(transa), int(transb), C.c_int64(M), C.c_int64(N), C.c_int64(K),
                                   C.c_float(alpha), _p(A, _f), C.c_int64(sa), _p(B, _f), C.c_int64(sb),
                                   C.c_float(0.0), _p(Cm, _f), C.c_int64(M * N), C.c_int64(batch))
    return Cm


def fused_parallel_gemm(A, W, bias, P, transa=False, transb=False, alpha=1.0, beta=1.0):
    A, W = f32(A), f32(W)
    M, K = (A.shape[1], A.shape[0]) if transa else A.shape
    N = (W.shape[0] // P) if transb else W.shape[1]
    Y = np.empty((P * M, N), np.float32)
    brow = 1
    if bias is not None:
        bias = f32(bias)
        brow = 1 if bias.ndim == 1 else M
    lib().orc_fused_parallel_gemm(int(transa), int(transb), P, C.c_int64(M), C.c_int64(N), C.c_int64(K),
                                  C.c_float(alpha), _p(A, _f), _p(W, _f), C.c_float(beta), _p(bias, _f),
                                  C.c_int64(brow), _p(Y, _f))
    return Y


def dice(x, gamma, mean, var, nosqrt=False):
    x = f32(x)
    c = x.shape[-1]
    y = np.empty_like(x)
    lib().orc_dice(_p(x, _f), C.c_int64(x.size // c), C.c_int64(c), _p(f32(gamma), _f), _p(f32(mean), _f),
                   _p(f32(var), _f), int(nosqrt), _p(y, _f))
    return y


def prelu(x, w):
    x, w = f32(x), f32(w).ravel()
    y = np.empty_like(x)
    lib().orc_prelu(_p(x, _f), C.c_int64(x.size), _p(w, _f), C.c_int64(w.size), _p(y, _f))
    return y


def sigmoid(x):
    x = f32(x)
    y = np.empty_like(x)
    lib().orc_sigmoid(_p(x, _f), C.c_int64(x.size), _p(y, _f))
    return y


def softmax(x, axis=1):
    x = f32(x)
    n = int(np.prod(x.shape[:axis], dtype=np.int64))
    c = x.shape[axis]
    w = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    y = np.empty_like(x)
    lib().orc_softmax(_p(x, _f), C.c_int64(n), C.c_int64(c), C.c_int64(w), _p(y, _f))
    return y


def batchnorm(x, gamma, beta, mean, var, eps=0.001, nosqrt=False):
    x = f32(x)
    y = np.empty_like(x)
    lib().orc_batchnorm(_p(x, _f), C.c_int64(x.size), C.c_int64(x.shape[-1]), _p(f32(gamma), _f),
                        _p(f32(beta), _f), _p(f32(mean), _f), _p(f32(var), _f), C.c_float(eps),
                        int(nosqrt), _p(y, _f))
    return y


def fuse(x1, x2):
    x1, x2 = f32(x1), f32(x2)
    ym = max(x1.shape[0], x2.shape[0])
    y = np.empty((ym, x1.shape[1] + x2.shape[1]), np.float32)
    lib().orc_fuse(_p(x1, _f), C.c_int64(x1.shape[0]), C.c_int64(x1.shape[1]), _p(x2, _f),
                   C.c_int64(x2.shape[0]), C.c_int64(x2.shape[1]), _p(y, _f))
    return y


def din_attention(q, k, w, act=2, seq_len=None, use_softmax=False, want_scores=False):
    """w: dict with W0,b0,W1,b1,W2,b2 and (for dice) g0,m0,v0,g1,m1,v1."""
    q, k = f32(q), f32(k)
    n, d = q.shape
    T = k.shape[0]
    keep = {n_: f32(w[n_]) if w.get(n_) is not None else None for n_, _ in AttW._fields_}
    aw = AttW(**{n_: _p(v, _f) for n_, v in keep.items()})
    h0, h1 = keep["W0"].shape[1], keep["W1"].shape[1]
    out = np.empty((n, d), np.float32)
    sc = np.empty((n, T), np.float32) if want_scores else None
    lib().orc_din_attention(_p(q, _f), C.c_int64(n), _p(k, _f), C.c_int64(T), d, h0, h1, C.byref(aw),
                            act, T if seq_len is None else int(seq_len), int(use_softmax), _p(out, _f),
                            _p(sc, _f))
    return (out, sc) if want_scores else out


def gru(x, h2h, i2h, h2h_bias, i2h_bias):
    x = f32(x)
    if x.ndim == 2:
        x = x[None]
    B, T, H = x.shape
    y = np.empty_like(x)
    lib().orc_gru(_p(x, _f), C.c_int64(B), C.c_int64(T), H, _p(f32(i2h), _f), _p(f32(h2h), _f),
                  _p(f32(i2h_bias), _f), _p(f32(h2h_bias), _f), _p(y, _f))
    return y


def augru(x, att, Wg, bg, Wc, bc):
    x, att = f32(x), f32(att)
    B, T, H = x.shape
    y = np.empty_like(x)
    lib().orc_augru(_p(x, _f), _p(att, _f), C.c_int64(B), C.c_int64(T), H, _p(f32(Wg), _f),
                    _p(f32(bg), _f), _p(f32(Wc), _f), _p(f32(bc), _f), _p(y, _f))
    return y


def route(ids, shards):
    ids = np.ascontiguousarray(ids, dtype=np.int64)
    owner = np.empty(ids.shape, np.int32)
    local = np.empty(ids.shape, np.int64)
    lib().orc_route(_p(ids, _i64), C.c_int64(ids.size), int(shards), _p(owner, _i32), _p(local, _i64))
    return owner, local


# ---------------------------------------------------------------------------
# The reference sparse store itself (compiled from the reference sources).
_ref = None


def ref_lib():
    """Returns the CDLL or None when oracle/_ref was never built."""
    global _ref
    if _ref is None:
        # the reference's whole CPU library when it was built (it contains the sparse store too), else the
        # sparse store alone; one process loads one of them, never both (each registers the reference's puller)
        path = os.path.join(ORACLE_DIR, "_ref", "libblaze_cpu.so")
        if not os.path.exists(path):
            path = os.path.join(ORACLE_DIR, "_ref", "libqed_ref.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
        _ref.ref_qed_open.restype = C.c_void_p
        _ref.ref_qed_open.argtypes = [C.c_char_p]
        _ref.ref_qed_close.argtypes = [C.c_void_p]
    return _ref


class RefStore:
    """QuickEmbeddingDict over fp32 tables given as {name: (keys, weights)}."""

    def __init__(self, tables, path):
        L = ref_lib()
        assert L is not None, "oracle/_ref/libqed_ref.so is not built"
        names = list(tables)
        n = len(names)
        c_names = (C.c_char_p * n)(*[s.encode() for s in names])
        dims = (C.c_int * n)()
        nrows = (C.c_int64 * n)()
        keyp = (_i64 * n)()
        wp = (_f * n)()
        self._keep = []
        for t, name in enumerate(names):
            keys, w = tables[name]
            keys = np.ascontiguousarray(keys, dtype=np.int64)
            w = f32(w)
            self._keep += [keys, w]
            dims[t], nrows[t] = w.shape[1], w.shape[0]
            keyp[t], wp[t] = _p(keys, _i64), _p(w, _f)
        rc = L.ref_qed_build(path.encode(), n, c_names, dims, nrows, keyp, wp)
        assert rc == 0, "ref_qed_build failed: %d" % rc
        self.h = L.ref_qed_open(path.encode())
        assert self.h, "ref_qed_open failed"
        self.dims = {name: tables[name][1].shape[1] for name in names}

    def get(self, table, keys, values, key_num, items):
        """Same item dicts as embedding_pool (assign_stride unsupported: reference layout only)."""
        L = ref_lib()
        dim = self.dims.get(table, items[0].get("dim", 1))
        keys = np.ascontiguousarray(keys, dtype=np.int64)
        values = f32(values)
        key_num = np.ascontiguousarray(key_num, dtype=np.int32)
        n = len(items)
        udf = (C.c_int * n)(*[it["udf"] for it in items])
        td = (C.c_int * n)(*[it.get("trunc_dir", 1) for it in items])
        tn = (C.c_int * n)(*[it.get("trunc_num", 0) for it in items])
        outs = (_f * n)()
        strides = (C.c_int64 * n)()
        for k, it in enumerate(items):
            o = it["out"]
            outs[k] = C.cast(o.ctypes.data + 4 * it.get("col", 0), _f)
            strides[k] = o.shape[1]
        return L.ref_qed_get(C.c_void_p(self.h), table.encode(), dim, _p(keys, _i64), _p(values, _f),
                             _p(key_num, _i32), C.c_int64(len(key_num)), n, udf, td, tn, outs, strides)

    def close(self):
        if self.h:
            ref_lib().ref_qed_close(C.c_void_p(self.h))
            self.h = None
