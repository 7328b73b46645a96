#!/usr/bin/env python3
"""Turn the reference's operator test nets into one compact JSON fixture.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py <reference checkout>

The reference's operator tests are text-proto NetDefs whose inputs are
ConstantFill ops and whose expected outputs are NetDef-level args
(blaze/blaze/test/operator/operator_test_common.h:19-84). This script parses
the CPU variants of the nets that touch the inference hot path and stores
them as plain data: {net: {ops: [...], expected: {output: {shape, values}}}}.
The result, tests/golden/blaze_op_fixtures.json, pins both the CPU oracle
(tests/test_oracle_golden.py) and the CUDA operators (tests/test_gpu_*.py).
"""
import glob
import json
import os
import re
import sys

TOKEN = re.compile(r'\s*(?:(#[^\n]*)|("(?:[^"\\]|\\.)*")|([{}:,])|([^\s{}:,#"]+))')


def tokenize(text):
    pos, out = 0, []
    while pos < len(text):
        m = TOKEN.match(text, pos)
        if not m:
            if text[pos:].strip() == "":
                break
            raise ValueError("bad text-proto at %d: %r" % (pos, text[pos:pos + 30]))
        pos = m.end()
        if m.group(1):
            continue
        if m.group(2) is not None:
            # protobuf text strings use C escapes
            out.append(("s", m.group(2)[1:-1].encode("latin1").decode("unicode_escape")))
        elif m.group(3):
            out.append((m.group(3), None))
        else:
            out.append(("w", m.group(4)))
    return out


def parse_message(toks, i, top=False):
    """Returns ({field: [values]}, next index)."""
    msg = {}
    while i < len(toks):
        kind, val = toks[i]
        if kind == "}":
            if top:
                raise ValueError("unbalanced }")
            return msg, i + 1
        if kind == ",":
            i += 1
            continue
        if kind != "w":
            raise ValueError("expected field name, got %r" % (toks[i],))
        name = val
        i += 1
        if toks[i][0] == ":":
            i += 1
        if toks[i][0] == "{":
            sub, i = parse_message(toks, i + 1)
            msg.setdefault(name, []).append(sub)
        else:
            k, v = toks[i]
            i += 1
            if k == "w":
                try:
                    v = int(v)
                except ValueError:
                    try:
                        v = float(v)
                    except ValueError:
                        pass
            msg.setdefault(name, []).append(v)
    return msg, i


def parse_text_proto(text):
    msg, _ = parse_message(tokenize(text), 0, top=True)
    return msg


def arg_to_plain(arg):
    out = {}
    for key in ("i", "f", "s"):
        if key in arg:
            out[key] = arg[key][0]
    for key in ("ints", "floats", "strings"):
        if key in arg:
            out[key] = arg[key]
    return out


def net_to_plain(net):
    ops = []
    for op in net.get("op", []):
        ops.append({
            "name": op.get("name", [""])[0],
            "type": op["type"][0],
            "input": op.get("input", []),
            "output": op.get("output", []),
            "arg": {a["name"][0]: arg_to_plain(a) for a in op.get("arg", [])},
        })
    args = {a["name"][0]: arg_to_plain(a) for a in net.get("arg", [])}
    expected = {}
    for eo in net.get("external_output", []):
        name = eo["name"][0]
        if name in args and name + "_shape" in args:
            vals = args[name].get("floats", args[name].get("ints"))
            expected[name] = {"shape": args[name + "_shape"]["ints"], "values": vals,
                              "dtype": eo.get("dtype", [1])[0]}
    return {"ops": ops, "expected": expected}


HOT_PATH_DIRS = [
    "op/gemm", "op/matmul", "op/dice", "op/prelu", "op/sigmoid", "op/softmax",
    "op/batch_normalization", "op/fuse", "op/concat", "op/elementwise", "op/reduce_sum",
    "op/slice", "op/split",
    "fused_op/fused_parallel_gemm", "fused_op/fused_parallel_matmul",
    "fused_op/fused_parallel_mul", "fused_op/fused_parallel_mul_reducesum",
    "fused_op/fused_slice_concat",
    "op/pruned_gemm",
]
# GRU: the reference ships 19 shapes; the small ones are enough to pin the gate math.
GRU_KEEP = re.compile(r"gru_test_(\d+)_(\d+)_(\d+)_cpu\.conf$")


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("XDL_REFERENCE", "")
    if not os.path.isdir(os.path.join(ref, "blaze")):
        sys.exit("usage: make_golden.py <root of the reference checkout>   (or set XDL_REFERENCE)")
    root = os.path.join(ref, "blaze/blaze/test/utest_data/operator")
    out = {}
    for d in HOT_PATH_DIRS:
        for path in sorted(glob.glob(os.path.join(root, d, "*_cpu.conf"))):
            key = os.path.relpath(path, root)
            out[key] = net_to_plain(parse_text_proto(open(path).read()))
    for path in sorted(glob.glob(os.path.join(root, "op/gru", "*_cpu.conf"))):
        m = GRU_KEEP.search(path)
        if m and int(m.group(1)) * int(m.group(2)) * int(m.group(3)) <= 64:
            out[os.path.relpath(path, root)] = net_to_plain(parse_text_proto(open(path).read()))
    emb = os.path.join(root, "sparse_op/embedding/embedding_v1.conf")
    if os.path.exists(emb):
        out["sparse_op/embedding/embedding_v1.conf"] = net_to_plain(parse_text_proto(open(emb).read()))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "blaze_op_fixtures.json")
    with open(dst, "w") as f:
        json.dump(out, f, separators=(",", ":"), sort_keys=True)
    print("wrote %s: %d nets, %d bytes" % (dst, len(out), os.path.getsize(dst)))


if __name__ == "__main__":
    main()
