"""One-time consolidation of `nn.ModuleList` experts into the fused tensors the grouped-GEMM path consumes, with
checkpoints that keep the per-expert layout.

The reference sketched this for Qwen3-MoE and gave it up ("consolidating params into tensor. OOMs",
scattermoe/utils/replace_moe.py:97-208): its `assemble_weights` (:105-126) stacked every expert's weights while the
originals were still alive, and its `state_dict` override (:149-167) split the fused tensors back into
`experts.{i}.{gate,up,down}_proj.weight`. The same three pieces here:

  * `consolidate_experts` copies one expert at a time into preallocated fused parameters and releases that expert's
    storage before touching the next, so the peak is the fused tensors plus ONE expert, not twice the layer;
  * `ConsolidatedExperts` holds `gate_up_proj (E, 2*I, H)` (activated "gate" half first) and `down_proj (E, H, I)`
    and runs the whole expert MLP as one autograd node (`expert_mlp`);
  * its state-dict hooks write per-expert keys on save and accept per-expert OR fused keys on load, so checkpoints
    stay interchangeable with the un-consolidated model.

`moe_block_forward` is the block forward of the reference's sketch (:171-206): router linear, fp32 softmax, top-k,
optional renormalisation, experts; here the router prologue is the fused `route_topk` kernel.
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from .. import _lib
from .. import activation as _act
from ..parallel_experts import expert_mlp, flatten_sort_count, parallel_linear
from ..routing import route_topk

# (gate, up, down) attribute names of one expert MLP: current Qwen / Llama-style, and Mixtral's older w1 / w3 / w2
QWEN_NAMES = ("gate_proj", "up_proj", "down_proj")
MIXTRAL_NAMES = ("w1", "w3", "w2")


class ConsolidatedExperts(nn.Module):
    """Fused-tensor replacement for a ModuleList of gated expert MLPs (`down(act(gate(x)) * up(x))`, no biases)."""

    def __init__(self, num_experts: int, hidden_size: int, intermediate_size: int, act_fn, names: Sequence[str] = QWEN_NAMES,
                 dtype=None, device=None):
        super().__init__()
        self.num_experts, self.hidden_size, self.intermediate_size = num_experts, hidden_size, intermediate_size
        self.act_fn = act_fn
        self.names = tuple(names)
        self.gate_up_proj = nn.Parameter(torch.empty(num_experts, 2 * intermediate_size, hidden_size, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(num_experts, hidden_size, intermediate_size, dtype=dtype, device=device))
        self._register_state_dict_hook(ConsolidatedExperts._split_on_save)
        self._register_load_state_dict_pre_hook(self._merge_on_load)

    def extra_repr(self):
        return "num_experts={}, hidden_size={}, intermediate_size={}".format(self.num_experts, self.hidden_size,
                                                                             self.intermediate_size)

    # ---- checkpoints keep the per-expert layout (replace_moe.py:149-167) ---------------------------------------
    @staticmethod
    def _split_on_save(module, state_dict, prefix, local_metadata):
        gate_name, up_name, down_name = module.names
        fused_up, fused_down = state_dict.pop(prefix + "gate_up_proj"), state_dict.pop(prefix + "down_proj")
        inter = module.intermediate_size
        for i in range(module.num_experts):
            state_dict["%s%d.%s.weight" % (prefix, i, gate_name)] = fused_up[i, :inter]
            state_dict["%s%d.%s.weight" % (prefix, i, up_name)] = fused_up[i, inter:]
            state_dict["%s%d.%s.weight" % (prefix, i, down_name)] = fused_down[i]
        return state_dict

    def _merge_on_load(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        if prefix + "gate_up_proj" in state_dict and prefix + "down_proj" in state_dict:
            return                                           # already fused
        gate_name, up_name, down_name = self.names
        first = "%s0.%s.weight" % (prefix, gate_name)
        if first not in state_dict:
            return                                           # nothing of ours: the regular loader reports what is missing
        ref = state_dict[first]
        fused_up = torch.empty((self.num_experts, 2 * self.intermediate_size, self.hidden_size), dtype=ref.dtype,
                               device=ref.device)
        fused_down = torch.empty((self.num_experts, self.hidden_size, self.intermediate_size), dtype=ref.dtype,
                                 device=ref.device)
        inter = self.intermediate_size
        for i in range(self.num_experts):
            keys = ["%s%d.%s.weight" % (prefix, i, n) for n in (gate_name, up_name, down_name)]
            absent = [k for k in keys if k not in state_dict]
            if absent:
                error_msgs.append("ConsolidatedExperts: checkpoint lacks %s" % ", ".join(absent))
                return
            fused_up[i, :inter].copy_(state_dict.pop(keys[0]))
            fused_up[i, inter:].copy_(state_dict.pop(keys[1]))
            fused_down[i].copy_(state_dict.pop(keys[2]))
        state_dict[prefix + "gate_up_proj"] = fused_up
        state_dict[prefix + "down_proj"] = fused_down

    # ---- forward: the signature of the fused expert blocks of current transformers releases ---------------------
    def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
                routing=None) -> torch.Tensor:
        shape = hidden_states.shape
        tokens = hidden_states.reshape(-1, shape[-1])
        _lib.require_cuda(tokens, "hidden_states")
        k = top_k_index.shape[-1]
        if routing is None:
            routing = flatten_sort_count(top_k_index.reshape(tokens.size(0), k), num_experts=self.num_experts)
        gates = top_k_weights.reshape(tokens.size(0), k).to(tokens.dtype)
        code = _act.resolve_activation(self.act_fn) if _act.FUSE else None
        if code is None:
            up = parallel_linear(tokens, self.gate_up_proj.transpose(2, 1), k, *routing, grouped_in=False, grouped_out=True)
            gate_half, linear_half = up.chunk(2, dim=-1)
            out = parallel_linear(self.act_fn(gate_half) * linear_half, self.down_proj.transpose(2, 1), 1, *routing,
                                  grouped_in=True, grouped_out=False, gates=gates)
        else:
            out = expert_mlp(tokens, self.gate_up_proj.transpose(2, 1), self.down_proj.transpose(2, 1), gates, k,
                             *routing, _act.LAYOUT_GLU_FIRST, code)
        return out.view(shape)


def consolidate_experts(experts: nn.ModuleList, names: Sequence[str] = QWEN_NAMES, act_fn=None) -> ConsolidatedExperts:
    """Build the fused module from a ModuleList of expert MLPs, releasing each expert's weights as soon as they have
    been copied (the ModuleList is left holding empty parameters and should be discarded by the caller)."""
    if len(experts) == 0:
        raise AssertionError("consolidate_experts: empty ModuleList")
    gate_name, up_name, down_name = names
    first = experts[0]
    for n in names:
        lin = getattr(first, n, None)
        if not isinstance(lin, nn.Linear) or lin.bias is not None:
            raise AssertionError("consolidate_experts: expert.%s must be a bias-free nn.Linear" % n)
    inter, hidden = getattr(first, gate_name).weight.shape
    w = getattr(first, gate_name).weight
    fused = ConsolidatedExperts(len(experts), hidden, inter, act_fn if act_fn is not None else getattr(first, "act_fn", None),
                                names, dtype=w.dtype, device=w.device)
    with torch.no_grad():
        for i, expert in enumerate(experts):
            for n, dst in ((gate_name, fused.gate_up_proj[i, :inter]), (up_name, fused.gate_up_proj[i, inter:]),
                           (down_name, fused.down_proj[i])):
                lin = getattr(expert, n)
                if lin.weight.shape != dst.shape:
                    raise AssertionError("consolidate_experts: expert %d %s has shape %s, expected %s"
                                         % (i, n, tuple(lin.weight.shape), tuple(dst.shape)))
                dst.copy_(lin.weight)
                lin.weight = nn.Parameter(torch.empty(0, dtype=w.dtype, device=w.device), requires_grad=False)   # release
    requires_grad = w.requires_grad
    fused.gate_up_proj.requires_grad_(requires_grad)
    fused.down_proj.requires_grad_(requires_grad)
    return fused


def consolidate_moe_block(block: nn.Module, experts_attr: str = "experts", names: Sequence[str] = QWEN_NAMES) -> nn.Module:
    """Replace `block.<experts_attr>` (a ModuleList) by its consolidated form, in place. Checkpoint keys of the block
    are unchanged (`<experts_attr>.{i}.<name>.weight`)."""
    experts = getattr(block, experts_attr)
    if isinstance(experts, ConsolidatedExperts):
        return block
    setattr(block, experts_attr, consolidate_experts(experts, names))
    return block


def moe_block_forward(block: nn.Module, hidden_states: torch.Tensor, gate_attr: str = "gate", experts_attr: str = "experts",
                      top_k: int = None, norm_topk_prob: bool = None):
    """Sparse-MoE block forward over consolidated experts (the reference's sketch, replace_moe.py:171-206): returns
    (final_hidden_states in the input's shape, router_logits (T, E)). `top_k` / `norm_topk_prob` default to the
    block's attributes of those names (Mixtral renormalises always, Qwen3 by configuration)."""
    experts = getattr(block, experts_attr)
    if not isinstance(experts, ConsolidatedExperts):
        raise AssertionError("moe_block_forward: consolidate the block's experts first (consolidate_moe_block)")
    shape = hidden_states.shape
    tokens = hidden_states.reshape(-1, shape[-1])
    router_logits = getattr(block, gate_attr)(tokens)
    k = top_k if top_k is not None else getattr(block, "top_k")
    renorm = norm_topk_prob if norm_topk_prob is not None else bool(getattr(block, "norm_topk_prob", True))
    gates, ids, routing = route_topk(router_logits, k, "softmax_topk", renormalize=renorm)
    out = experts(tokens, ids, gates.to(tokens.dtype), routing=routing)
    return out.view(shape), router_logits
