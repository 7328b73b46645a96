"""The graph-fusion pass of the host runtime on the op-by-op DIN graph: host logic, no GPU needed (a model is
parsed and rewritten when it is loaded; only creating a predictor needs a device)."""
import numpy as np

import pkg


def _load(dtype, optimize, mutate=None):
    pkg.load()
    from x_deeplearning_b200 import blaze_api as api, din_netdef, workloads
    model = workloads.din_model(0, item_rows=300, cate_rows=50, user_rows=100, emb_sigma=0.5)
    text, _ = din_netdef.build_unfused(model, dtype=dtype, device_type=1)
    if mutate:
        text = mutate(text)
    mgr = api.PredictorManager()
    mgr.load_model_text(text, optimize=optimize)
    types = mgr.op_types()
    mgr.close()
    return types


def test_unfused_fp16_graph_becomes_two_fused_operators():
    plain = _load(12, False)
    fused = _load(12, True)
    for t in ("Sub", "Mul", "BroadcastTo", "MatMul", "Fuse", "ReduceSum", "Softmax", "Gemm", "Dice"):
        assert t in plain
    assert fused.count("DinAttention") == 1 and fused.count("DinTower") == 1
    for t in ("Sub", "Mul", "BroadcastTo", "MatMul", "Fuse", "ReduceSum", "Softmax", "Gemm", "Dice"):
        assert t not in fused, t
    # what is left: the two Embedding operators, the reshapes and the concat that build k and q, constants
    assert sorted(set(fused)) == ["Concat", "ConstantFill", "DinAttention", "DinTower", "Embedding", "Reshape"]
    # the constants only the removed nodes read (reshape targets) are gone; the 12 + 12 weights stay
    assert fused.count("ConstantFill") == 12 + 12 + 3
    assert fused.index("DinAttention") < fused.index("DinTower")


def test_fp32_graph_is_left_alone():
    fused = _load(1, True)
    assert "DinAttention" not in fused and "DinTower" not in fused
    assert "Sub" in fused and "Fuse" in fused


def test_a_blob_read_outside_the_pattern_blocks_the_fusion():
    # a second consumer of the attention MLP's first activation: the attention sub-graph must stay, and with
    # it the tower (its att input no longer comes from the fused unit)
    def extra_reader(text):
        return text.replace('external_output {', 'op { type: "Sigmoid" name: "spy" input: "att_y0" output: "spy" }\n'
                            'external_output { name: "spy" dtype: 12 }\nexternal_output {', 1)
    fused = _load(12, True, extra_reader)
    assert "DinAttention" not in fused and "DinTower" not in fused
    assert "Sub" in fused and "MatMul" in fused
