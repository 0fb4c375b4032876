"""Hugging Face MoE blocks routed through the B200 grouped-GEMM path.

Mirrors the reference's scattermoe/utils/replace_moe.py: importing this module swaps
`GptOssExperts.forward` (:21-55) and `GraniteMoeHybridMoE.forward` (:62-93) for versions built on
`parallel_linear` + `flatten_sort_count`; the swap is logged on first use (:8-17) and a failure to patch is
logged and swallowed (:56-57, :94-95).

Two differences from the reference text, both needed to run against current transformers releases:
  * gpt_oss: `routing_weights` may be the dense (T, E) score matrix the reference gathers from (:26) or the
    already selected (T, k) scores newer routers return; it is gathered only in the first case.
  * granitemoehybrid: the reference returns `(layer_output, router_logits)` (:93); releases whose own forward
    returns the tensor alone get the tensor alone, otherwise the caller's residual add breaks.
Inputs that are not on a CUDA device are handed to the original Hugging Face forward: this package has no
CPU implementation.
"""
import inspect
import logging

import torch

from .. import _lib
from .. import activation as _act
from ..parallel_experts import expert_mlp, flatten_sort_count, parallel_linear
from ..routing import route_topk

PATCHED = {}      # class name -> original forward


def replace_function(cls, fun_name):
    """Class-method swap that announces itself the first time the replacement runs (replace_moe.py:8-17)."""
    def decorator(fun):
        PATCHED[cls.__name__] = getattr(cls, fun_name)

        def _announce_then_call(*args, **kwargs):
            logging.info("Replacing `%s.%s` with %s:%s", cls.__name__, fun_name, fun.__code__.co_filename,
                         fun.__name__)
            setattr(cls, fun_name, fun)
            return fun(*args, **kwargs)
        setattr(cls, fun_name, _announce_then_call)
        return fun
    return decorator


def gpt_oss_glu(gate_up: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    """Clamped SwiGLU on interleaved gate/up columns (replace_moe.py:39-43)."""
    if _act.FUSE and _lib.on_device(gate_up) and gate_up.dim() == 2:
        return _act.fused_activation(gate_up, _act.LAYOUT_GPT_OSS, _act.ACT_SILU, alpha, limit)
    gate, up = gate_up[..., ::2], gate_up[..., 1::2]
    gate = gate.clamp(min=None, max=limit)
    up = up.clamp(min=-limit, max=limit)
    return (up + 1) * (gate * torch.sigmoid(gate * alpha))


try:
    from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts

    @replace_function(cls=GptOssExperts, fun_name='forward')
    def gpt_oss_forward(self, hidden_states: torch.Tensor, router_indices=None, routing_weights=None) -> torch.Tensor:
        if not _lib.on_device(hidden_states):
            return PATCHED['GptOssExperts'](self, hidden_states, router_indices=router_indices,
                                            routing_weights=routing_weights)
        batch_size = hidden_states.shape[0]
        tokens = hidden_states.reshape(-1, self.hidden_size)
        k = router_indices.shape[1]
        if routing_weights.shape[-1] == self.num_experts:
            # dense (T, E) scores, the layout the reference expects (k == E is read this way too)
            selected = torch.gather(routing_weights, dim=1, index=router_indices)
        else:
            selected = routing_weights                                                  # already (T, k)
        routing = flatten_sort_count(router_indices.flatten(), num_experts=self.num_experts)
        if _act.FUSE:
            out = expert_mlp(tokens, self.gate_up_proj, self.down_proj, selected.to(tokens.dtype), k, *routing,
                             _act.LAYOUT_GPT_OSS, _act.ACT_SILU, up_biases=self.gate_up_proj_bias,
                             down_biases=self.down_proj_bias, alpha=self.alpha, limit=self.limit)
        else:
            gate_up = parallel_linear(tokens, self.gate_up_proj, k, *routing,
                                      expert_biases=self.gate_up_proj_bias, grouped_in=False, grouped_out=True)
            gated = gpt_oss_glu(gate_up, self.alpha, self.limit)
            out = parallel_linear(gated, self.down_proj, 1, *routing,
                                  expert_biases=self.down_proj_bias, grouped_in=True, grouped_out=False,
                                  gates=selected.to(tokens.dtype))
        return out.view(batch_size, -1, self.hidden_size)
except Exception:  # transformers absent or without this model
    logging.info("Failed to replace GptOssExperts")


try:
    from transformers.models.granitemoehybrid.modeling_granitemoehybrid import GraniteMoeHybridMoE

    def _original_returns_tuple(fn) -> bool:
        try:
            src = inspect.getsource(fn)
        except (OSError, TypeError):
            return True
        return any(line.strip().startswith("return") and "," in line for line in src.splitlines())

    GRANITE_RETURNS_ROUTER_LOGITS = _original_returns_tuple(GraniteMoeHybridMoE.forward)

    @replace_function(cls=GraniteMoeHybridMoE, fun_name='forward')
    def granite_moe_forward(self, layer_input):
        if not _lib.on_device(layer_input):
            return PATCHED['GraniteMoeHybridMoE'](self, layer_input)
        bsz, length, emb_size = layer_input.size()
        tokens = layer_input.reshape(-1, emb_size)
        # top-k routing decision (replace_moe.py:67-71: fp32 softmax over the experts, top-k, renormalise) fused with
        # the routing bookkeeping: one kernel from the logits to ids, gates and the sort's histograms
        router_logits = self.router.layer(tokens)
        probs, selected_experts, routing = route_topk(router_logits, self.router.top_k, "softmax_topk", renormalize=True)
        probs = probs.to(tokens.dtype)
        # experts: the FIRST half of the up-projection is the activated one here (replace_moe.py:76-83)
        code = _act.resolve_activation(self.activation) if _act.FUSE else None
        if code is None:
            up = parallel_linear(tokens, self.input_linear.weight.transpose(2, 1), self.router.top_k, *routing,
                                 grouped_in=False, grouped_out=True)
            gate_half, linear_half = up.chunk(2, dim=-1)
            hidden = self.activation(gate_half) * linear_half
            layer_output = parallel_linear(hidden, self.output_linear.weight.transpose(2, 1), 1, *routing,
                                           grouped_in=True, grouped_out=False, gates=probs)
        else:
            layer_output = expert_mlp(tokens, self.input_linear.weight.transpose(2, 1),
                                      self.output_linear.weight.transpose(2, 1), probs, self.router.top_k, *routing,
                                      _act.LAYOUT_GLU_FIRST, code)
        layer_output = layer_output.view(bsz, length, emb_size)
        if GRANITE_RETURNS_ROUTER_LOGITS:
            return layer_output, router_logits
        return layer_output
except Exception:
    logging.info("Failed to replace GraniteMoeHybridMoE")


# Blocks the reference does not patch (its Qwen3 attempt is commented out, replace_moe.py:97-208, written for
# releases that kept experts in a ModuleList and needed a weight consolidation pass). Current transformers releases
# store these experts as fused 3-D parameters already -- gate_up_proj (E, 2*I, H) with the activated "gate" half
# first, down_proj (E, H, I) -- which is exactly what `parallel_linear` consumes, so the patch is the granite one
# without a router: forward(hidden_states (T, H), top_k_index (T, k), top_k_weights (T, k)) -> (T, H).
def _fused_glu_experts_forward(cls_name):
    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> torch.Tensor:
        if not _lib.on_device(hidden_states):
            return PATCHED[cls_name](self, hidden_states, top_k_index, top_k_weights)
        shape = hidden_states.shape
        tokens = hidden_states.reshape(-1, shape[-1])
        k = top_k_index.shape[-1]
        routing = flatten_sort_count(top_k_index.reshape(tokens.size(0), k), num_experts=self.num_experts)
        code = _act.resolve_activation(self.act_fn) if _act.FUSE else None
        if code is None:
            up = parallel_linear(tokens, self.gate_up_proj.transpose(2, 1), k, *routing, grouped_in=False, grouped_out=True)
            gate_half, linear_half = up.chunk(2, dim=-1)
            hidden = self.act_fn(gate_half) * linear_half
            out = parallel_linear(hidden, self.down_proj.transpose(2, 1), 1, *routing, grouped_in=True,
                                  grouped_out=False, gates=top_k_weights.reshape(tokens.size(0), k).to(tokens.dtype))
        else:
            out = expert_mlp(tokens, self.gate_up_proj.transpose(2, 1), self.down_proj.transpose(2, 1),
                             top_k_weights.reshape(tokens.size(0), k).to(tokens.dtype), k, *routing,
                             _act.LAYOUT_GLU_FIRST, code)
        return out.view(shape)
    forward.__name__ = "fused_glu_experts_forward_" + cls_name
    return forward


for _module, _cls_name in (("transformers.models.qwen3_moe.modeling_qwen3_moe", "Qwen3MoeExperts"),
                           ("transformers.models.mixtral.modeling_mixtral", "MixtralExperts")):
    try:
        import importlib
        _cls = getattr(importlib.import_module(_module), _cls_name)
        _src = inspect.getsource(_cls)
        if not all(word in _src for word in ("gate_up_proj", "down_proj", "top_k_index", "top_k_weights")):
            raise ImportError("%s does not keep fused expert tensors in this transformers release" % _cls_name)
        replace_function(cls=_cls, fun_name='forward')(_fused_glu_experts_forward(_cls_name))
    except Exception:
        logging.info("Failed to replace %s", _cls_name)
