"""The CPU oracle against the golden vectors produced by running the reference package
(tests/golden/make_golden.py). Pins every oracle function before any GPU test relies on it."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import scattermoe_oracle as oracle  # noqa: E402
from util import as_dtype, assert_close, golden_names, load_golden, segments_equal_as_sets  # noqa: E402


@pytest.mark.parametrize("name", golden_names("sort_"))
def test_flatten_sort_count(name):
    g = load_golden(name)
    se, ss, off = oracle.flatten_sort_count(g["expert_idxs"], g["E"])
    assert torch.equal(se, g["sorted_expert_idxs"])
    assert torch.equal(off, g["expert_offsets"])
    if g["reference_was_stable"]:
        assert torch.equal(ss, g["sorted_scattered_idxs"])
    else:  # the reference's torch.sort is not stable for this size: equal per expert as sets
        assert segments_equal_as_sets(ss, g["sorted_scattered_idxs"], off)
    assert torch.equal(oracle.offsets_from_sorted(se, g["E"]), g["expert_offsets"])


@pytest.mark.parametrize("name", golden_names("s2s_"))
def test_scatter2scatter(name):
    g = load_golden(name)
    X, W, b = as_dtype(g, g["X"]), as_dtype(g, g["W"]), as_dtype(g, g.get("b"))
    # the row order of grouped inputs/outputs is the order of the index tensors the reference produced
    se, ss = g["sorted_expert_idxs"], g["sorted_scattered_idxs"]
    Y = oracle.scatter2scatter(X, W, se, ss, g["k"], b=b, x_grouped=g["x_grouped"], y_grouped=g["y_grouped"])
    assert_close(name, Y, g["Y"], g["bf16"])


@pytest.mark.parametrize("name", golden_names("group_"))
def test_group(name):
    g = load_golden(name)
    ss = g["sorted_scattered_idxs"]
    Y = oracle.group(as_dtype(g, g["A"]), ss, coeff=as_dtype(g, g.get("coeff")), fan_out=g["k"])
    assert_close(name, Y, g["Y"], g["bf16"])


@pytest.mark.parametrize("name", golden_names("gbw_"))
def test_group_bwd_w(name):
    g = load_golden(name)
    off = g["expert_offsets"]
    DW, Db = oracle.group_bwd_W(as_dtype(g, g["DY"]), as_dtype(g, g["X"]), off, g["E"], has_bias="Db" in g)
    assert_close(name + ".DW", DW, g["DW"], g["bf16"])
    if "Db" in g:
        assert_close(name + ".Db", Db, g["Db"], g["bf16"])
    counts = torch.bincount(g["expert_idxs"].flatten(), minlength=g["E"])
    assert (DW[counts == 0] == 0).all(), "experts without rows must give exact zeros"


def _mlp_case(g, activation, w1_key="param.experts.weight", w2_key="param.output_experts.weight"):
    dt = torch.bfloat16 if g["bf16"] else torch.float32
    w1 = g[w1_key].permute(0, 2, 1)      # stored (E, out, in) -> logical (E, in, out)
    w2 = g[w2_key].permute(0, 2, 1)
    b1, b2 = g.get("param.experts.bias"), g.get("param.output_experts.bias")
    return oracle.moe_mlp_forward_backward(g["X"], g["expert_p"], g["expert_idxs"], w1, w2, b1, b2, activation, g["DY"],
                                           compute_dtype=torch.float32), dt


@pytest.mark.parametrize("name,act", [
    ("mlp_gelu_fp32", "gelu"), ("mlp_gelu_fp32_bias", "gelu"), ("mlp_gelu_fp32_T1", "gelu"),
    ("glumlp_silu_fp32", "glu"), ("glumlp_silu_bf16", "glu"), ("mlp_gelu_bf16", "gelu")])
def test_dense_loop_matches_reference_mlp(name, act):
    g = load_golden(name)
    activation = oracle.act_gelu if act == "gelu" else oracle.act_glu_second_half
    out, dt = _mlp_case(g, activation)
    bf16 = g["bf16"]
    assert_close(name + ".Y", out["y"], g["Y"], bf16)
    assert_close(name + ".dX", out["d_x"], g["dX"], bf16)
    assert_close(name + ".dg", out["d_expert_p"], g["d_expert_p"], bf16)
    assert_close(name + ".dW1", out["d_w1"].permute(0, 2, 1), g["grad.experts.weight"], bf16)
    assert_close(name + ".dW2", out["d_w2"].permute(0, 2, 1), g["grad.output_experts.weight"], bf16)
    if "d_b1" in out:
        assert_close(name + ".db1", out["d_b1"], g["grad.experts.bias"], bf16)
        assert_close(name + ".db2", out["d_b2"], g["grad.output_experts.bias"], bf16)


def test_parallel_linear_orchestration_matches_reference_mlp():
    """Forward and backward of the two-layer MLP assembled from the oracle's ParallelLinear restatement
    (the kernel-level functions, not the dense loop) against the reference's own outputs."""
    g = load_golden("mlp_gelu_fp32_bias")
    E, k = g["E"], g["k"]
    se, ss, off = oracle.flatten_sort_count(g["expert_idxs"], E)
    w1 = g["param.experts.weight"].permute(0, 2, 1)
    w2 = g["param.output_experts.weight"].permute(0, 2, 1)
    b1, b2 = g["param.experts.bias"], g["param.output_experts.bias"]
    x, p = g["X"], g["expert_p"]
    h, _ = oracle.parallel_linear_forward(x, w1, k, se, ss, off, b1, None, False, True)
    hp = h.clone().requires_grad_()
    a = oracle.act_gelu(hp)
    y, expanded = oracle.parallel_linear_forward(a.detach(), w2, 1, se, ss, off, b2, p, True, False)
    assert_close("Y", y, g["Y"], False)
    d_a, d_w2, d_b2, d_p = oracle.parallel_linear_backward(g["DY"], a.detach(), w2, 1, se, ss, off, b2, p, expanded, True, False)
    (d_h,) = torch.autograd.grad(a, hp, d_a)
    d_x, d_w1, d_b1, _ = oracle.parallel_linear_backward(d_h, x, w1, k, se, ss, off, b1, None, None, False, True)
    assert_close("dX", d_x, g["dX"], False)
    assert_close("dg", d_p, g["d_expert_p"], False)
    assert_close("dW1", d_w1.permute(0, 2, 1), g["grad.experts.weight"], False)
    assert_close("dW2", d_w2.permute(0, 2, 1), g["grad.output_experts.weight"], False)
    assert_close("db1", d_b1, g["grad.experts.bias"], False)
    assert_close("db2", d_b2, g["grad.output_experts.bias"], False)


def test_hf_gpt_oss_golden():
    g = load_golden("hf_gpt_oss_experts")
    hs = g["hidden_states"]
    T = hs.shape[0] * hs.shape[1]
    out = oracle.moe_mlp_forward_backward(hs.reshape(T, -1), g["routing_weights_topk"], g["router_indices"],
                                          g["param.gate_up_proj"], g["param.down_proj"], g["param.gate_up_proj_bias"],
                                          g["param.down_proj_bias"], oracle.act_gpt_oss, g["DY"].reshape(T, -1))
    assert_close("Y", out["y"].reshape(hs.shape), g["Y"], False)
    assert_close("dX", out["d_x"].reshape(hs.shape), g["d_hidden_states"], False)
    assert_close("dg", out["d_expert_p"], g["d_routing_weights_topk"], False)
    assert_close("dW1", out["d_w1"], g["grad.gate_up_proj"], False)
    assert_close("dW2", out["d_w2"], g["grad.down_proj"], False)
    assert_close("db1", out["d_b1"], g["grad.gate_up_proj_bias"], False)
    assert_close("db2", out["d_b2"], g["grad.down_proj_bias"], False)


def test_hf_granite_golden():
    g = load_golden("hf_granitemoehybrid_moe")
    x = g["layer_input"]
    T = x.shape[0] * x.shape[1]
    xt = x.reshape(T, -1)
    logits = xt @ g["param.router.layer.weight"].t()
    assert_close("router_logits", logits, g["router_logits"], False)
    p = torch.softmax(logits.float(), dim=1)
    p, idx = torch.topk(p, 2, dim=-1)
    p = p / p.sum(-1, keepdim=True)
    out = oracle.moe_mlp_forward_backward(xt, p, idx, g["param.input_linear.weight"].permute(0, 2, 1),
                                          g["param.output_linear.weight"].permute(0, 2, 1), None, None,
                                          oracle.act_glu_first_half, g["DY"].reshape(T, -1))
    assert_close("Y", out["y"].reshape(x.shape), g["Y"], False)
    assert_close("dW1", out["d_w1"].permute(0, 2, 1), g["grad.input_linear.weight"], False)
    assert_close("dW2", out["d_w2"].permute(0, 2, 1), g["grad.output_linear.weight"], False)


@pytest.mark.parametrize("name", golden_names("single_"))
def test_single2scatter(name):
    """The single-token kernel (kernels/single.py) as run by the reference itself."""
    g = load_golden(name)
    y = oracle.single2scatter(g["X"], g["W"], g["expert_idxs"])     # W stored as (E, K, N) values
    assert_close(name, y, g["Y"], False)
