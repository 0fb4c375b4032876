"""Drop-in surface: the names, signatures, defaults, parameter names/shapes and import side effects of the
reference package (scattermoe/__init__.py:1-15, parallel_experts.py, mlp.py, kernels/ops.py, utils/replace_moe.py)."""
import inspect

import torch
from torch import nn

import scattermoe_b200 as scattermoe


def params(fn):
    return [(n, p.default) for n, p in inspect.signature(fn).parameters.items()]


def test_package_exports():
    for name in ["flatten_sort_count", "parallel_linear", "ParallelExperts", "parallel_experts", "kernels", "mlp", "utils"]:
        assert hasattr(scattermoe, name), name
        assert name in scattermoe.__all__
    assert hasattr(scattermoe.kernels, "ops") and hasattr(scattermoe.utils, "replace_moe")
    ops = scattermoe.kernels.ops
    assert ops.BLOCK_M == 128 and ops.ALLOW_TF32 is True
    assert hasattr(scattermoe.mlp, "MLP") and hasattr(scattermoe.mlp, "GLUMLP")


def test_function_signatures_match_reference():
    E = inspect.Parameter.empty
    assert params(scattermoe.flatten_sort_count) == [("expert_idxs", E), ("num_experts", E)]
    assert params(scattermoe.parallel_linear) == [
        ("inputs", E), ("expert_weights", E), ("k", E), ("sorted_expert_idxs", E), ("sorted_scattered_idxs", E),
        ("expert_offsets", E), ("expert_biases", None), ("gates", None), ("grouped_in", False), ("grouped_out", False)]
    ops = scattermoe.kernels.ops
    # reference positional order, then this build's optional extras
    assert params(ops.scatter2scatter)[:9] == [
        ("X", E), ("W", E), ("sorted_expert_idxs", E), ("sorted_scattered_idxs", E), ("k", E), ("b", None),
        ("x_grouped", False), ("y_grouped", False), ("out", None)]
    assert params(ops.group_bwd_W)[:5] == [("DY", E), ("X", E), ("expert_offsets", E), ("E", E), ("has_bias", False)]
    assert params(ops.group) == [("A", E), ("sorted_expert_idxs", E), ("coeff", None), ("fan_out", 1), ("out", None)]
    fwd = params(scattermoe.ParallelExperts.forward)
    assert fwd == [("self", E), ("inputs", E), ("k", E), ("sorted_expert_idxs", E), ("sorted_scattered_idxs", E),
                   ("expert_offsets", E), ("gates", None), ("grouped_in", False), ("grouped_out", False)]
    assert [n for n, _ in params(scattermoe.parallel_experts.ParallelLinear.forward)] == [
        "ctx", "x", "expert_weights", "k", "sorted_expert_idxs", "sorted_scattered_idxs", "expert_offsets",
        "expert_biases", "gates", "grouped_in", "grouped_out"]


def test_module_parameters_and_repr():
    torch.manual_seed(0)
    m = scattermoe.mlp.MLP(16, 24, 4, 9, bias=True, activation=nn.GELU())
    assert m.top_k == 4                                        # min(top_k, num_experts), mlp.py:23
    sd = m.state_dict()
    assert {k: tuple(v.shape) for k, v in sd.items()} == {
        "experts.weight": (4, 24, 16), "experts.bias": (4, 24),
        "output_experts.weight": (4, 16, 24), "output_experts.bias": (4, 16)}
    assert torch.count_nonzero(m.experts.bias) == 0             # zeros init, parallel_experts.py:169-170
    assert 0.01 < m.experts.weight.std().item() < 0.03         # N(0, 0.02)
    assert "k=4" in repr(m) and "num_experts=4, input_size=16, output_size=24" in repr(m)
    g = scattermoe.mlp.GLUMLP(16, 24, 4, 2)
    assert tuple(g.experts.weight.shape) == (4, 48, 16) and g.experts.bias is None
    assert isinstance(g.activation, nn.SiLU)
    # the reference's example constructs this and prints it (examples/molora.py)
    assert "MLP" in repr(scattermoe.mlp.MLP(input_size=64, hidden_size=8, activation=nn.Identity(), num_experts=16, top_k=2))


def test_hf_patches_are_installed_on_import():
    rm = scattermoe.utils.replace_moe
    from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts
    from transformers.models.granitemoehybrid.modeling_granitemoehybrid import GraniteMoeHybridMoE
    assert {"GptOssExperts", "GraniteMoeHybridMoE"} <= set(rm.PATCHED)
    assert GptOssExperts.forward is not rm.PATCHED["GptOssExperts"]
    assert GraniteMoeHybridMoE.forward is not rm.PATCHED["GraniteMoeHybridMoE"]
    assert callable(rm.gpt_oss_forward) and callable(rm.granite_moe_forward)


def test_hf_cpu_inputs_use_the_original_forward():
    """The patched blocks hand non-CUDA inputs back to Hugging Face's own code instead of failing."""
    from transformers.models.granitemoehybrid.modeling_granitemoehybrid import GraniteMoeHybridMoE
    from transformers.models.granitemoehybrid.configuration_granitemoehybrid import GraniteMoeHybridConfig
    cfg = GraniteMoeHybridConfig(hidden_size=64, intermediate_size=48, num_local_experts=8, num_experts_per_tok=2,
                                 num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                                 shared_intermediate_size=32)
    moe = GraniteMoeHybridMoE(cfg)
    out = moe(torch.randn(1, 5, 64))
    out = out[0] if isinstance(out, tuple) else out
    assert out.shape == (1, 5, 64)
