"""The DIN-style model as a Blaze NetDef for the host runtime (Predictor API).

Graph (fp16 model): two Embedding operators as in the shipped DIN graph
(blaze/tools/example_model/din/model/graph_ulf.txt: a user-side op with the uid
block and the two kAssign behaviour blocks, an ad-side op with the item|category
block), Reshape x2 + Concat to k [R, T, 36], then the fused DinAttention and
DinTowerInput operators and the tower Gemm -> Dice, Gemm -> Dice, Gemm -> Softmax
(the Dice nodes are folded into the Gemm epilogues by LoadModel's fusion pass).
"""
import numpy as np

from . import blaze_api as api

F16, F32, I32, I64 = 12, 1, 2, 10


def _fg(name, table, dim):
    return 'feature_group_config { feature_group: "%s" table_name: "%s" dim: %d }\n' % (name, table, dim)


def _item(fg, udf, trunc_num=None):
    extra = "" if trunc_num is None else " trunc_num: %d" % trunc_num
    return '  embedding_block_config_item { feature_group: "%s" udf_type: %d%s }\n' % (fg, udf, extra)


def build(model, fused_tower=True):
    """Returns (netdef_text, input_names) for `model` (workloads.din_model). With `fused_tower` the tower is
    the single DinTower operator (output fp32); without it the tower stays a chain of reference operators
    (DinTowerInput, PrunedGemm, Dice, Gemm, Dice, Gemm, Softmax; output fp16)."""
    D = model["dims"]
    e, d, T, G = D["emb"], D["d"], D["T"], D["user_groups"]
    users = ["u%d" % g for g in range(G)]
    triple = lambda n: [n + ".ids", n + ".values", n + ".segments"]
    ops = []
    # user-side Embedding: uid block (G kSum items), mid_list and cat_list kAssign blocks
    conf = "".join(_fg(u, "user%d" % g, e) for g, u in enumerate(users))
    conf += _fg("mid_list", "item", e) + _fg("cat_list", "cate", e)
    conf += "block_config {\n" + "".join(_item(u, 0) for u in users) + "}\n"
    conf += "block_config {\n" + _item("mid_list", 2, T) + "}\n"
    conf += "block_config {\n" + _item("cat_list", 2, T) + "}\n"
    user_in = sum([triple(u) for u in users], []) + triple("mid_list") + triple("cat_list")
    ops.append(api.op_text("Embedding", user_in, ["uid_emb", "mid_list_emb", "cat_list_emb"], {"embedding_config": conf},
                           "user_embedding"))
    conf = _fg("mid", "item", e) + _fg("cat", "cate", e) + "block_config {\n" + _item("mid", 0) + _item("cat", 0) + "}\n"
    ops.append(api.op_text("Embedding", triple("mid") + triple("cat"), ["ad_emb"], {"embedding_config": conf}, "ad_embedding"))
    ops.append(api.op_text("Reshape", ["mid_list_emb"], ["mid_list_3d"], {"shape": [-1, T, e]}))
    ops.append(api.op_text("Reshape", ["cat_list_emb"], ["cat_list_3d"], {"shape": [-1, T, e]}))
    ops.append(api.op_text("Concat", ["mid_list_3d", "cat_list_3d"], ["his_emb"], {"axis": 2}))
    a = model["att"]
    names = []
    for n in ("W0", "b0", "W1", "b1", "W2", "b2", "g0", "m0", "v0", "g1", "m1", "v1"):
        ops.append(api.constant_text("att_" + n, a[n], F16))
        names.append("att_" + n)
    ops.append(api.op_text("DinAttention", ["ad_emb", "his_emb"] + names, ["att"], {"act": 2}))
    tw = model["tower"]
    feeds = []
    for n in users + ["mid_list", "cat_list", "mid", "cat"]:
        feeds += [(n + ".ids", I64), (n + ".values", F16), (n + ".segments", I32)]
    if fused_tower:
        consts = []
        for i, key in ((1, "dice1"), (2, "dice2"), (3, None)):
            group = [("W%d" % i, tw["W%d" % i]), ("b%d" % i, tw["b%d" % i])]
            if key:
                group += [("%s%d" % (n, i), arr) for n, arr in zip(("g", "m", "v"), tw[key])]
            for name, arr in group:
                ops.append(api.constant_text("t_" + name, arr, F16))
                consts.append("t_" + name)
        ops.append(api.op_text("DinTower", ["uid_emb", "ad_emb", "his_emb", "att"] + consts, ["output"]))
        return api.netdef_text(ops, feeds, [("output", F32)], name="din"), [n for n, _ in feeds]
    # first tower layer as a PrunedGemm: the columns that are equal for all candidates of a request
    # ([user | his_sum]) are one operand, the per-candidate columns the other
    ops.append(api.op_text("DinTowerInput", ["uid_emb", "ad_emb", "his_emb", "att"], ["tower_user", "tower_cand"]))
    from .din import split_tower_rows
    rows_u, rows_c = split_tower_rows(G * e, d)

    def padded(rows):
        ld = (len(rows) + 7) // 8 * 8                         # rows of the zero padding columns of the operand
        W = np.zeros((ld, tw["W1"].shape[1]), np.float32)
        W[:len(rows)] = tw["W1"][rows]
        return W
    for name, arr in (("W1u", padded(rows_u)), ("W1c", padded(rows_c)), ("b1", tw["b1"]), ("W2", tw["W2"]), ("b2", tw["b2"]),
                      ("W3", tw["W3"]), ("b3", tw["b3"])):
        ops.append(api.constant_text("t_" + name, arr, F16))
    for i, key in ((1, "dice1"), (2, "dice2")):
        for n, arr in zip(("g", "m", "v"), tw[key]):
            ops.append(api.constant_text("t_%s%d" % (n, i), arr, F16))
    ops.append(api.op_text("PrunedGemm", ["tower_user", "tower_cand", "t_W1u", "t_W1c", "t_b1"], ["h1"]))
    ops.append(api.op_text("Dice", ["h1", "t_g1", "t_m1", "t_v1"], ["y1"]))
    ops.append(api.op_text("Gemm", ["y1", "t_W2", "t_b2"], ["h2"]))
    ops.append(api.op_text("Dice", ["h2", "t_g2", "t_m2", "t_v2"], ["y2"]))
    ops.append(api.op_text("Gemm", ["y2", "t_W3", "t_b3"], ["logit"]))
    ops.append(api.op_text("Softmax", ["logit"], ["output"], {"axis": 1}))
    return api.netdef_text(ops, feeds, [("output", F16)], name="din"), [n for n, _ in feeds]


def build_unfused(model, dtype=F32, device_type=0):
    """The same model for ONE request with reference operators only, composed the way the shipped DIN graph is
    (blaze/tools/example_model/din/model/graph_ulf.txt: Sub, Mul, BroadcastTo x2, Concat, three Gemm layers with
    their activations, the weighted sum as a batched MatMul, ReduceSum, Mul, Concat, Fuse, the tower Gemm / Dice
    chain and Softmax). This is the graph the reference's own CPU operators run in the benchmark's reference arm,
    and the graph the fusion pass of the host runtime turns back into DinAttention + DinTower.
    Returns (netdef_text, input_names); output "output" [n_cand, 2] in `dtype`."""
    D = model["dims"]
    e, d, T, G = D["emb"], D["d"], D["T"], D["user_groups"]
    users = ["u%d" % g for g in range(G)]
    triple = lambda n: [n + ".ids", n + ".values", n + ".segments"]
    O = api.op_text
    ops = []

    def reshape(x, y, shape):
        # the reference's Reshape reads the new shape from an int32 tensor (blaze/blaze/operator/op/reshape_op.h:17-50)
        ops.append(api.constant_text(y + "_shape", np.asarray(shape), I32))
        ops.append(O("Reshape", [x, y + "_shape"], [y]))
    conf = "".join(_fg(u, "user%d" % g, e) for g, u in enumerate(users))
    conf += _fg("mid_list", "item", e) + _fg("cat_list", "cate", e)
    conf += "block_config {\n" + "".join(_item(u, 0) for u in users) + "}\n"
    conf += "block_config {\n" + _item("mid_list", 2, T) + "}\n"
    conf += "block_config {\n" + _item("cat_list", 2, T) + "}\n"
    user_in = sum([triple(u) for u in users], []) + triple("mid_list") + triple("cat_list")
    ops.append(O("Embedding", user_in, ["uid_emb", "mid_list_emb", "cat_list_emb"], {"embedding_config": conf}, "user_embedding"))
    conf = _fg("mid", "item", e) + _fg("cat", "cate", e) + "block_config {\n" + _item("mid", 0) + _item("cat", 0) + "}\n"
    ops.append(O("Embedding", triple("mid") + triple("cat"), ["ad_emb"], {"embedding_config": conf}, "ad_embedding"))
    reshape("mid_list_emb", "mid_list_3d", [1, -1, e])
    reshape("cat_list_emb", "cat_list_3d", [1, -1, e])
    ops.append(O("Concat", ["mid_list_3d", "cat_list_3d"], ["his_emb"], {"axis": 2}))          # [1, T, d]
    reshape("ad_emb", "item_emb", [-1, 1, d])                  # [n, 1, d]
    # attention unit, rows 7-16 of the shipped graph
    ops.append(O("Sub", ["item_emb", "his_emb"], ["sub_emb"]))                                 # [n, T, d]
    ops.append(O("Mul", ["item_emb", "his_emb"], ["mul_emb"]))
    ops.append(O("BroadcastTo", ["his_emb", "sub_emb"], ["b_his_emb"]))
    ops.append(O("BroadcastTo", ["item_emb", "sub_emb"], ["b_item_emb"]))
    ops.append(O("Concat", ["b_item_emb", "b_his_emb", "sub_emb", "mul_emb"], ["att_in"], {"axis": 2}))   # [n, T, 4d]
    a = model["att"]
    for n in ("W0", "b0", "W1", "b1", "W2", "b2", "g0", "m0", "v0", "g1", "m1", "v1"):
        ops.append(api.constant_text("att_" + n, a[n], dtype))
    ops.append(O("Gemm", ["att_in", "att_W0", "att_b0"], ["att_h0"]))
    ops.append(O("Dice", ["att_h0", "att_g0", "att_m0", "att_v0"], ["att_y0"]))
    ops.append(O("Gemm", ["att_y0", "att_W1", "att_b1"], ["att_h1"]))
    ops.append(O("Dice", ["att_h1", "att_g1", "att_m1", "att_v1"], ["att_y1"]))
    ops.append(O("Gemm", ["att_y1", "att_W2", "att_b2"], ["att_s"]))                           # [n, T, 1]
    reshape("att_s", "att_w", [-1, 1, T])                      # [n, 1, T]
    ops.append(O("MatMul", ["att_w", "his_emb"], ["att_3d"]))                                  # [n, 1, d]
    reshape("att_3d", "att", [-1, d])
    # tower input, rows 17-22
    ops.append(O("ReduceSum", ["his_emb"], ["his_sum"], {"axis": 1, "keepdims": 0}))           # [1, d]
    ops.append(O("Mul", ["ad_emb", "his_sum"], ["mul_item"]))
    ops.append(O("Sub", ["ad_emb", "his_sum"], ["sub_item"]))
    ops.append(O("BroadcastTo", ["his_sum", "ad_emb"], ["b_his_sum"]))
    ops.append(O("Concat", ["ad_emb", "b_his_sum", "mul_item", "att", "sub_item"], ["cand_side"], {"axis": 1}))
    ops.append(O("Fuse", ["uid_emb", "cand_side"], ["tower_in"]))
    tw = model["tower"]
    for i, key in ((1, "dice1"), (2, "dice2"), (3, None)):
        ops.append(api.constant_text("t_W%d" % i, tw["W%d" % i], dtype))
        ops.append(api.constant_text("t_b%d" % i, tw["b%d" % i], dtype))
        if key:
            for n, arr in zip(("g", "m", "v"), tw[key]):
                ops.append(api.constant_text("t_%s%d" % (n, i), arr, dtype))
    ops.append(O("Gemm", ["tower_in", "t_W1", "t_b1"], ["h1"]))
    ops.append(O("Dice", ["h1", "t_g1", "t_m1", "t_v1"], ["y1"]))
    ops.append(O("Gemm", ["y1", "t_W2", "t_b2"], ["h2"]))
    ops.append(O("Dice", ["h2", "t_g2", "t_m2", "t_v2"], ["y2"]))
    ops.append(O("Gemm", ["y2", "t_W3", "t_b3"], ["logit"]))
    ops.append(O("Softmax", ["logit"], ["output"], {"axis": 1}))
    feeds = []
    for n in users + ["mid_list", "cat_list", "mid", "cat"]:
        feeds += [(n + ".ids", I64), (n + ".values", dtype), (n + ".segments", I32)]
    return api.netdef_text(ops, feeds, [("output", dtype)], device_type=device_type, name="din_unfused"), [n for n, _ in feeds]


def register_tables(mgr, model):
    mgr.load_sparse(None, "b200_sparse_puller")
    mgr.add_table("item", model["item"], F16)
    mgr.add_table("cate", model["cate"], F16)
    for g, w in enumerate(model["user"]):
        mgr.add_table("user%d" % g, w, F16)


def feeds_of(model, req):
    """{feed name: numpy array} for one batch of requests (workloads.din_requests)."""
    D = model["dims"]
    R, n_cand = req["requests"], req["n_cand"]
    out = {}

    def put(name, ids, segments):
        out[name + ".ids"] = np.ascontiguousarray(ids, np.int64)
        out[name + ".values"] = np.ones(len(ids), np.float16)
        out[name + ".segments"] = np.ascontiguousarray(segments, np.int32)
    for g in range(D["user_groups"]):
        put("u%d" % g, req["user_ids"][:, g], np.ones(R, np.int32))
    put("mid_list", req["hist_item"], req["seq_len"])
    put("cat_list", req["hist_cate"], req["seq_len"])
    put("mid", req["cand_item"], np.ones(R * n_cand, np.int32))
    put("cat", req["cand_cate"], np.ones(R * n_cand, np.int32))
    return out
