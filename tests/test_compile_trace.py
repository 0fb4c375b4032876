"""Host-only check that torch.compile traces a whole layer, forward and backward, without a graph break.

No kernel runs here: the ctypes library is replaced by a recorder that answers "ok" to every call, and CPU tensors
stand in for device tensors. What is checked is the part that needs no GPU: every launch sits behind a registered
operator with a usable fake, nothing in between is untraceable, and the traced step issues the same C-ABI calls in
the same order as the eager step. Numerics under torch.compile are checked on the GPU
(tests/test_gpu_mlp.py::test_module_runs_under_torch_compile).
"""
import contextlib

import pytest
import torch
from torch import nn

import scattermoe_b200 as sm
from scattermoe_b200 import _lib


class RecordingLibrary:
    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        if name == "smoe_sort_count_workspace_bytes":
            return lambda *a: 1024

        def call(*args):
            self.calls.append(name)
            return 0
        return call


@pytest.fixture
def recorder(monkeypatch):
    rec = RecordingLibrary()
    monkeypatch.setattr(_lib, "load", lambda: rec)
    monkeypatch.setattr(_lib, "on_device", lambda t: True)
    monkeypatch.setattr(_lib, "stream_ptr", lambda dev: 0)
    monkeypatch.setattr(_lib, "status_word", lambda dev: torch.zeros(4, dtype=torch.int32))
    monkeypatch.setattr(torch.cuda, "device", lambda dev: contextlib.nullcontext())
    yield rec
    torch._dynamo.reset()


def _step(fn, module, x, p, idx, rec):
    rec.calls.clear()
    y = fn(x, p, idx)
    fwd = list(rec.calls)
    rec.calls.clear()
    grads = torch.autograd.grad(y, [x, p] + list(module.parameters()), torch.ones_like(y))
    return y.shape, [g.shape for g in grads], fwd, list(rec.calls)


@pytest.mark.parametrize("kind,dtype,bias", [("glu", torch.bfloat16, True), ("glu", torch.float32, False),
                                             ("mlp", torch.bfloat16, False)])
def test_layer_traces_as_one_graph(recorder, kind, dtype, bias):
    torch.manual_seed(0)
    if kind == "glu":
        module = sm.mlp.GLUMLP(64, 48, 4, 2, bias=bias).to(dtype)
    else:
        module = sm.mlp.MLP(64, 48, 4, 2, bias=bias, activation=nn.GELU()).to(dtype)
    x = torch.randn(10, 64, dtype=dtype, requires_grad=True)
    p, idx = torch.topk(torch.softmax(torch.randn(10, 4), -1), 2)
    p = p.detach().to(dtype).requires_grad_()
    eager = _step(module, module, x, p, idx, recorder)
    compiled = torch.compile(module, backend="aot_eager", fullgraph=True)     # fullgraph: any graph break raises
    traced = _step(compiled, module, x, p, idx, recorder)
    assert traced[0] == eager[0] and traced[1] == eager[1]
    assert traced[2] == eager[2], (traced[2], eager[2])
    assert sorted(traced[3]) == sorted(eager[3]), (traced[3], eager[3])       # backward: same launches, any order
    assert "smoe_scatter2scatter" in eager[2] and "smoe_group_bwd_w" in eager[3]
    if dtype == torch.bfloat16:
        assert "smoe_scatter2scatter_act_bwd" in eager[3] and "smoe_activation_backward" not in eager[3]


@pytest.mark.parametrize("family", ["qwen3_moe", "gpt_oss"])
def test_patched_hugging_face_block_traces_as_one_graph(recorder, family):
    """The patched expert blocks (utils/replace_moe.py) are plain callers of parallel_linear: they trace whole too."""
    torch.manual_seed(0)
    w, idx = torch.topk(torch.softmax(torch.randn(12, 8), -1), 2)
    w = w.bfloat16()
    if family == "qwen3_moe":
        from transformers.models.qwen3_moe.configuration_qwen3_moe import Qwen3MoeConfig
        from transformers.models.qwen3_moe.modeling_qwen3_moe import Qwen3MoeExperts
        cfg = Qwen3MoeConfig(hidden_size=64, moe_intermediate_size=48, num_experts=8, num_experts_per_tok=2,
                             num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, intermediate_size=64)
        block = Qwen3MoeExperts(cfg).bfloat16()
        x = torch.randn(12, 64, dtype=torch.bfloat16, requires_grad=True)
        call = lambda f: f(x, idx, w)
    else:
        from transformers.models.gpt_oss.configuration_gpt_oss import GptOssConfig
        from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts
        cfg = GptOssConfig(hidden_size=64, intermediate_size=48, num_local_experts=8, num_experts_per_tok=2,
                           num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1)
        block = GptOssExperts(cfg).bfloat16()
        x = torch.randn(1, 12, 64, dtype=torch.bfloat16, requires_grad=True)
        call = lambda f: f(x, router_indices=idx, routing_weights=w)
    call(block)                       # first call swaps the class method in (not part of the trace)
    recorder.calls.clear()
    call(block)
    eager = list(recorder.calls)
    recorder.calls.clear()
    y = call(torch.compile(block, backend="aot_eager", fullgraph=True))
    assert list(recorder.calls) == eager and "smoe_scatter2scatter_act" in eager
    recorder.calls.clear()
    y.sum().backward()
    # backward: two weight gradients, the fused (input gradient of the down-projection + activation gradient) launch
    # and the input gradient of the up-projection
    assert recorder.calls.count("smoe_group_bwd_w") == 2 and recorder.calls.count("smoe_scatter2scatter") == 1
    assert recorder.calls.count("smoe_scatter2scatter_act_bwd") == 1 and "smoe_activation_backward" not in recorder.calls
    if family == "qwen3_moe":       # no down-projection bias: the gate gradient comes out of the fused launch
        assert "smoe_gate_grad" not in recorder.calls and "smoe_gate_grad_from_partials" in recorder.calls
