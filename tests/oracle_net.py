"""Runs a fixture net (tests/golden/blaze_op_fixtures.json) on the CPU oracle.

Compute ops go through oracle/liboracle.so (tests/orc.py); pure data movement
(concat, slice, broadcast) is numpy indexing. Mirrors what the reference's
TestOperatorOutput does with a text-proto NetDef
(blaze/blaze/test/operator/operator_test_common.h:19-84)."""
import numpy as np

import orc

DTYPES = {1: np.float32, 2: np.int32, 10: np.int64, 12: np.float32}


def _arg(op, name, default=None, key="i"):
    a = op["arg"].get(name)
    if a is None:
        return default
    for k in (key, "i", "f", "s", "ints", "floats"):
        if k in a:
            return a[k]
    return default


def constant_fill(op):
    shape = op["arg"]["shape"]["ints"]
    dt = DTYPES.get(_arg(op, "dtype", 1), np.float32)
    v = op["arg"]["value"]
    vals = v.get("floats", v.get("ints", [v.get("f", v.get("i", 0))]))
    a = np.array(vals, dtype=dt)
    n = int(np.prod(shape))
    if a.size == 1 and n != 1:
        a = np.full(n, a[0], dtype=dt)
    return a.reshape(shape)


def _batched_matmul(a, b, ta, tb):
    """numpy-broadcast batched matmul expressed through the strided-batched oracle GEMM,
    as BroadcastGemm_NxN / BatchedBroadcastGemm_NxN do (blaze/blaze/math/broadcast.h:156-381)."""
    M, K = (a.shape[-1], a.shape[-2]) if ta else (a.shape[-2], a.shape[-1])
    N = b.shape[-2] if tb else b.shape[-1]
    na = int(np.prod(a.shape[:-2], dtype=np.int64))
    nb = int(np.prod(b.shape[:-2], dtype=np.int64))
    batch = max(na, nb)
    sa = 0 if na == 1 and batch > 1 else M * K
    sb = 0 if nb == 1 and batch > 1 else K * N
    lead = a.shape[:-2] if na >= nb else b.shape[:-2]
    return orc.gemm_strided_batched(a, sa, b, sb, M, N, K, batch, ta, tb).reshape(tuple(lead) + (M, N))


def run_op(op, env):
    t = op["type"]
    x = [env[n] for n in op["input"]]
    if t == "ConstantFill":
        return [constant_fill(op)]
    if t == "Gemm":
        a = x[0]
        bias = x[2] if len(x) > 2 else None
        ta, tb = bool(_arg(op, "transA", 0)), bool(_arg(op, "transB", 0))
        alpha, beta = _arg(op, "alpha", 1.0, "f"), _arg(op, "beta", 1.0, "f")
        if a.ndim == 3:
            ys = [orc.gemm_op(a[i], x[1], bias, ta, tb, alpha, beta) for i in range(a.shape[0])]
            return [np.stack(ys)]
        return [orc.gemm_op(a, x[1], bias, ta, tb, alpha, beta)]
    if t == "PrunedGemm":
        return [orc.pruned_gemm(x[0], x[1], x[2], x[3], x[4] if len(x) > 4 else None,
                                _arg(op, "alpha", 1.0, "f"), _arg(op, "beta", 1.0, "f"))]
    if t == "FusedParallelGemm":
        return [orc.fused_parallel_gemm(x[0], x[1], x[2] if len(x) > 2 else None, _arg(op, "parallel_num"),
                                        bool(_arg(op, "transA", 0)), bool(_arg(op, "transB", 0)),
                                        _arg(op, "alpha", 1.0, "f"), _arg(op, "beta", 1.0, "f"))]
    if t == "MatMul":
        return [_batched_matmul(x[0], x[1], bool(_arg(op, "transA", 0)), bool(_arg(op, "transB", 0)))]
    if t == "FusedParallelMatMul":
        P = _arg(op, "parallel_num")
        a = x[0].reshape((P, -1) + x[0].shape[1:])
        b = x[1].reshape((P, -1) + x[1].shape[1:])
        outs = [_batched_matmul(a[p], b[p], bool(_arg(op, "transA", 0)), bool(_arg(op, "transB", 0)))
                for p in range(P)]
        return [np.concatenate(outs, axis=0)]
    if t == "Dice":
        return [orc.dice(x[0], x[1], x[2], x[3], bool(_arg(op, "nosqrt", 0)))]
    if t == "PRelu":
        return [orc.prelu(x[0], x[1])]
    if t == "Sigmoid":
        return [orc.sigmoid(x[0])]
    if t == "Softmax":
        return [orc.softmax(x[0], _arg(op, "axis", 1))]
    if t == "BatchNormalization":
        return [orc.batchnorm(x[0], x[1], x[2], x[3], x[4], _arg(op, "eps", 0.001, "f"),
                              bool(_arg(op, "nosqrt", 0)))]
    if t == "Fuse":
        return [orc.fuse(x[0], x[1])]
    if t == "GRU":
        return [orc.gru(x[0], x[1], x[2], x[3], x[4])]
    if t == "Concat":
        return [np.concatenate(x, axis=_arg(op, "axis", 1))]
    if t in ("Add", "Sub", "Mul", "Div", "Max", "Min", "Equal", "NotEqual"):
        f = {"Add": np.add, "Sub": np.subtract, "Mul": np.multiply, "Div": np.divide, "Max": np.maximum,
             "Min": np.minimum, "Equal": np.equal, "NotEqual": np.not_equal}[t]
        return [f(x[0], x[1]).astype(x[0].dtype)]
    if t == "BroadcastTo":
        return [np.broadcast_to(x[0], x[1].shape).copy()]
    if t == "Where":
        return [np.where(x[0] != 0, x[1], x[2]).astype(x[1].dtype)]
    if t == "ReduceSum":
        return [x[0].sum(axis=_arg(op, "axis", 0), keepdims=bool(_arg(op, "keepdims", 1)), dtype=np.float32)]
    if t == "Slice":
        idx = [slice(None)] * x[0].ndim
        idx[_arg(op, "axis", 1)] = slice(_arg(op, "start"), _arg(op, "end"))
        return [x[0][tuple(idx)].copy()]
    if t == "Split":
        axis = _arg(op, "axis", 0)
        sizes = op["arg"].get("split", {}).get("ints")
        n = len(op["output"])
        if sizes is None:
            sizes = [x[0].shape[axis] // n] * n
        cuts = np.cumsum(sizes)[:-1]
        return [p.copy() for p in np.split(x[0], cuts, axis=axis)]
    if t == "FusedSliceConcat":
        sa, ca = _arg(op, "slice_axis"), _arg(op, "concat_axis")
        parts = []
        for s, e in zip(op["arg"]["start"]["ints"], op["arg"]["end"]["ints"]):
            idx = [slice(None)] * x[0].ndim
            idx[sa] = slice(s, e)
            parts.append(x[0][tuple(idx)])
        return [np.concatenate(parts, axis=ca)]
    if t in ("FusedParallelMul", "FusedParallelMulReduceSum"):
        P = _arg(op, "parallel_num", 2)
        a = x[0].reshape((P, -1) + x[0].shape[1:])
        b = x[1].reshape((P, -1) + x[1].shape[1:])
        outs = []
        for p in range(P):
            m = (a[p] * b[p]).astype(np.float32)
            if t == "FusedParallelMulReduceSum":
                m = m.sum(axis=_arg(op, "axis", 0), keepdims=bool(_arg(op, "keepdims", 1)), dtype=np.float32)
                if m.ndim == 0 or not bool(_arg(op, "keepdims", 1)) and _arg(op, "axis", 0) == 0:
                    m = m.reshape((1,) + m.shape) if False else m
            outs.append(m)
        if t == "FusedParallelMulReduceSum" and not bool(_arg(op, "keepdims", 1)) and _arg(op, "axis", 0) == 0:
            return [np.concatenate([o.ravel() for o in outs])]
        return [np.concatenate(outs, axis=0)]
    raise NotImplementedError(t)


def run_net(net, feeds=None):
    env = dict(feeds or {})
    for op in net["ops"]:
        outs = run_op(op, env)
        for name, val in zip(op["output"], outs):
            env[name] = val
    return env
