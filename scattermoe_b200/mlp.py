"""MoE MLP modules with the reference's constructors, parameter names and forward signatures
(scattermoe/mlp.py: MLP :6-49, GLUMLP :51-95).

Both modules are two `ParallelExperts` (`experts`, `output_experts`) with an activation between them; they
differ only in the width of the first projection and in how the activation consumes it, so they share one
base class here.
"""
import torch
from torch import nn

from . import _lib
from . import activation as _act
from .parallel_experts import ParallelExperts, expert_mlp, flatten_sort_count


class _ExpertMLPBase(nn.Module):
    """Routing bookkeeping -> up-projection into expert-grouped rows -> `_activate` -> down-projection back
    to token order with the top-k gate-weighted sum."""

    up_factor = 1  # width of the first projection in units of hidden_size
    act_layout = _act.LAYOUT_PLAIN

    def __init__(self, input_size, hidden_size, num_experts, top_k, bias, activation):
        super().__init__()
        self.num_experts = num_experts
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.experts = ParallelExperts(num_experts, input_size, self.up_factor * hidden_size, bias=bias)
        self.output_experts = ParallelExperts(num_experts, hidden_size, input_size, bias=bias)
        self.top_k = min(top_k, self.num_experts)   # mlp.py:23
        self.activation = activation

    def extra_repr(self):
        return 'k={}'.format(self.top_k)

    def _activate(self, up: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward(self, x: torch.Tensor, expert_p: torch.Tensor, expert_idxs: torch.Tensor):
        lead = x.shape[:-1]
        tokens = x.view(-1, x.shape[-1])            # any leading shape, restored on return (mlp.py:30-31, :48)
        routing = flatten_sort_count(expert_idxs, num_experts=self.num_experts)
        code = _act.resolve_activation(self.activation) if _act.FUSE else None
        if code is not None and expert_p is not None and _lib.on_device(tokens):
            # the whole expert MLP as one autograd node: activation in the epilogue of the up-projection GEMM,
            # activation gradient in the epilogue of the down-projection's input-gradient GEMM (tensor-core cases;
            # separate one-pass kernels otherwise)
            y = expert_mlp(tokens, self.experts.weight.permute(0, 2, 1), self.output_experts.weight.permute(0, 2, 1),
                           expert_p.reshape(tokens.size(0), expert_idxs.shape[-1]), self.top_k, *routing, self.act_layout, code,
                           up_biases=self.experts.bias, down_biases=self.output_experts.bias)
        else:
            up = self.experts(tokens, self.top_k, *routing, grouped_out=True)
            hidden = self._activate(up)
            y = self.output_experts(hidden, 1, *routing, grouped_in=True, gates=expert_p)
        return y.view(*lead, y.size(-1))


class MLP(_ExpertMLPBase):
    """mlp.py:6-49. `activation` has no usable default in the reference either (None is not callable):
    always pass one, e.g. nn.GELU()."""

    up_factor = 1

    def __init__(self, input_size, hidden_size, num_experts, top_k, bias=False, activation=None):
        super().__init__(input_size, hidden_size, num_experts, top_k, bias, activation)

    def _activate(self, up):
        code = _act.resolve_activation(self.activation) if _act.FUSE else None
        if code is None or up.dim() != 2:
            return self.activation(up)
        return _act.fused_activation(up, _act.LAYOUT_PLAIN, code)


class GLUMLP(_ExpertMLPBase):
    """mlp.py:51-95. The first projection is 2*hidden wide; its SECOND half is the activated one:
    `h, gates = chunk(2)`, `act(gates) * h` (mlp.py:81-87)."""

    up_factor = 2
    act_layout = _act.LAYOUT_GLU_SECOND

    def __init__(self, input_size, hidden_size, num_experts, top_k, bias=False, activation=nn.SiLU()):
        super().__init__(input_size, hidden_size, num_experts, top_k, bias, activation)

    def _activate(self, up):
        code = _act.resolve_activation(self.activation) if _act.FUSE else None
        if code is None or up.dim() != 2:
            linear_half, gate_half = up.chunk(2, dim=-1)
            return self.activation(gate_half) * linear_half
        return _act.fused_activation(up, _act.LAYOUT_GLU_SECOND, code)
