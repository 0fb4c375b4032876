"""Autograd boundary of the expert linear layer; same surface as the reference's
scattermoe/parallel_experts.py (flatten_sort_count :14, ParallelLinear :25, parallel_linear :136,
ParallelExperts :148).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import _lib
from . import activation as _act
from . import kernels


def _sort_count_impl(flat: torch.Tensor, num_experts: int):
    _lib.require_cuda(flat, "expert_idxs")
    R = flat.numel()
    dev = flat.device
    lib = _lib.load()
    sorted_e = torch.empty(R, dtype=torch.int64, device=dev)
    sorted_idx = torch.empty(R, dtype=torch.int64, device=dev)
    offsets = torch.empty(num_experts, dtype=torch.int64, device=dev)
    ws_bytes = lib.smoe_sort_count_workspace_bytes(R, num_experts)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.smoe_sort_count(flat.data_ptr(), R, num_experts, sorted_e.data_ptr(), sorted_idx.data_ptr(),
                                 offsets.data_ptr(), ws.data_ptr(), ws_bytes, _lib.stream_ptr(dev))
    _lib.check(rc, "smoe_sort_count")
    return sorted_e, sorted_idx, offsets


@torch.library.custom_op("scattermoe_b200::sort_count", mutates_args={})
def sort_count_compileable(flat_expert_idxs: torch.Tensor, num_experts: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Traceable form; plays the role of the reference's scattermoe::bincount op (parallel_experts.py:6-12)."""
    return _sort_count_impl(flat_expert_idxs, num_experts)


@sort_count_compileable.register_fake
def _(flat_expert_idxs: torch.Tensor, num_experts: int):
    R = flat_expert_idxs.numel()
    dev = flat_expert_idxs.device
    return (torch.empty(R, dtype=torch.long, device=dev), torch.empty(R, dtype=torch.long, device=dev),
            torch.empty(num_experts, dtype=torch.long, device=dev))


def flatten_sort_count(expert_idxs: torch.Tensor, num_experts: int):
    """parallel_experts.py:14-21. Returns (sorted_expert_idxs, sorted_scattered_idxs, expert_offsets):
    expert ids ascending, the flat slot index `t*k+j` of every sorted entry in ascending order inside one
    expert (the stable order; the reference's torch.sort leaves ties unspecified), and the inclusive
    cumulative per-expert counts. One counting-sort pass on the device; no host synchronisation and no
    torch.compile needed."""
    with torch.no_grad():
        flat = expert_idxs.flatten()
        in_dtype = flat.dtype
        if in_dtype != torch.int64:
            flat = flat.to(torch.int64)
        flat = flat.contiguous()
        if torch.compiler.is_compiling():
            sorted_e, sorted_idx, offsets = sort_count_compileable(flat, num_experts)
        else:
            sorted_e, sorted_idx, offsets = _sort_count_impl(flat, num_experts)
        if in_dtype != torch.int64:
            sorted_e = sorted_e.to(in_dtype)
        return sorted_e, sorted_idx, offsets


# Un-grouped 16-bit inputs are first copied into expert order (one HBM pass, `kernels.ops.group`) so that the
# tensor-core kernels of the forward AND of the weight gradient read them with TMA; the copy is kept for
# backward, where the reference makes the same copy anyway (parallel_experts.py:99). Measured on B200 the
# TMA-fed kernels run ~2x faster than the cp.async row gather for the weight gradient. False: gather in-kernel.
GROUP_INPUT_COPY = True

# `ExpertMLP` without a down-projection bias: apply the gates to the hidden rows inside the fused up-projection kernel
# and take the gate gradient from the fused hidden-gradient kernel (no separate gate-weighting or gate-gradient pass).
# False: gate-weighted top-k sum after the down-projection and a separate gate-gradient kernel, as the reference does.
FUSE_GATES = True


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


class ParallelLinear(torch.autograd.Function):
    """parallel_experts.py:25-134, same argument order and return arity.

    Differences that are not visible in results: the top-k reductions are dedicated kernels instead of
    batched matmuls (:44-46, :79, :123); the expert-order copy of an un-grouped input that the reference makes
    in backward (:99) is made once in forward and shared by the forward GEMM and the weight gradient (see
    GROUP_INPUT_COPY; with it off both kernels gather the rows themselves and no copy exists); gradients
    nobody asked for are not computed.
    """

    @staticmethod
    def forward(ctx, x: torch.Tensor, expert_weights: torch.Tensor, k: int,
                sorted_expert_idxs: torch.Tensor, sorted_scattered_idxs: torch.Tensor,
                expert_offsets: torch.Tensor,
                expert_biases: Optional[torch.Tensor] = None,
                gates: Optional[torch.Tensor] = None,
                grouped_in: bool = False, grouped_out: bool = False):
        x = _rowmajor(x)
        x_in_expert_order = None
        if (not grouped_in and GROUP_INPUT_COPY and x.dtype in (torch.bfloat16, torch.float16)
                and x.size(1) % 8 == 0 and _lib.on_device(x)):
            x_in_expert_order = kernels.ops.group(x, sorted_scattered_idxs, fan_out=k)
            output = kernels.ops.scatter2scatter(
                X=x_in_expert_order, W=expert_weights, b=expert_biases, k=1,
                sorted_expert_idxs=sorted_expert_idxs, sorted_scattered_idxs=sorted_scattered_idxs,
                x_grouped=True, y_grouped=grouped_out, expert_offsets=expert_offsets)
        else:
            output = kernels.ops.scatter2scatter(
                X=x, W=expert_weights, b=expert_biases, k=k,
                sorted_expert_idxs=sorted_expert_idxs, sorted_scattered_idxs=sorted_scattered_idxs,
                x_grouped=grouped_in, y_grouped=grouped_out, expert_offsets=expert_offsets)
        if gates is not None:
            output_expanded = output.view(gates.size(0), gates.size(1), output.size(-1))
            output = kernels.ops.topk_reduce(output, gates, gates.size(0), gates.size(1))
        else:
            output_expanded = None
        ctx.save_for_backward(x, expert_weights, expert_biases, sorted_expert_idxs, sorted_scattered_idxs,
                              expert_offsets, gates, output_expanded, x_in_expert_order)
        ctx.grouped_in = grouped_in
        ctx.grouped_out = grouped_out
        ctx.k = k
        return output

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        (x, expert_weights, expert_biases, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
         gates, output_expanded, x_in_expert_order) = ctx.saved_tensors
        k = ctx.k
        grouped_in = ctx.grouped_in
        grouped_out = ctx.grouped_out
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = expert_biases is not None and ctx.needs_input_grad[6]
        need_g = gates is not None and ctx.needs_input_grad[7]
        grad_out = _rowmajor(grad_out)
        if grad_out.dtype != x.dtype:
            grad_out = grad_out.to(x.dtype)

        d_gates = None
        if gates is not None:
            T, gate_fan = gates.size(0), gates.size(1)
            expanded_flat = output_expanded.flatten(0, 1)
            if need_g:
                d_gates = kernels.ops.gate_grad(expanded_flat, grad_out, T, gate_fan).to(gates.dtype)
            gates_flat = gates.flatten()
            grouped_grad_out = expanded_flat   # storage reused below, as the reference does (:82)
        else:
            gates_flat = None
            gate_fan = 1
            grouped_grad_out = None

        d_input = d_weights = d_biases = None
        if need_x or need_w or need_b:
            if grouped_out:
                grouped_grad_out = grad_out
            else:
                # a traced backward must not write into a tensor saved by forward: allocate there instead of reusing
                grouped_grad_out = kernels.ops.group(
                    grad_out, sorted_scattered_idxs, fan_out=gate_fan, coeff=gates_flat,
                    out=None if torch.compiler.is_compiling() else grouped_grad_out)
            if need_w or need_b:
                x_rows_grouped = grouped_in or x_in_expert_order is not None
                d_weights, d_biases = kernels.ops.group_bwd_W(
                    DY=grouped_grad_out, X=x if grouped_in else (x_in_expert_order if x_rows_grouped else x),
                    expert_offsets=expert_offsets, E=expert_weights.size(0),
                    has_bias=expert_biases is not None,
                    x_gather_idx=None if x_rows_grouped else sorted_scattered_idxs,
                    fan_out=1 if x_rows_grouped else k)
            if need_x:
                d_expanded_input = kernels.ops.scatter2scatter(
                    X=grouped_grad_out, x_grouped=True, W=expert_weights.permute(0, 2, 1),
                    sorted_expert_idxs=sorted_expert_idxs, sorted_scattered_idxs=sorted_scattered_idxs,
                    k=1, y_grouped=grouped_in, expert_offsets=expert_offsets)
                if k == 1:
                    d_input = d_expanded_input
                else:
                    d_input = kernels.ops.topk_reduce(d_expanded_input, None, x.size(0), k)
        return (d_input, d_weights, None, None, None, None, d_biases, d_gates, None, None)


class ParallelLinearAct(torch.autograd.Function):
    """Up-projection into expert order followed by the activation, forward in ONE kernel (the activation runs in
    the epilogue of the tensor-core grouped GEMM); the reference runs `ParallelLinear` (grouped_out=True) and
    then PyTorch elementwise ops (scattermoe/mlp.py:35-41, :76-87). Backward: one activation-gradient kernel,
    then exactly the backward of `ParallelLinear`."""

    @staticmethod
    def forward(ctx, x, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, expert_biases,
                act_layout, act, alpha, limit):
        x = _rowmajor(x)
        x_src, kk, grouped = x, k, False
        if GROUP_INPUT_COPY and x.size(1) % 8 == 0 and x.dtype in (torch.bfloat16, torch.float16):
            x_src, kk, grouped = kernels.ops.group(x, sorted_scattered_idxs, fan_out=k), 1, True
        res = kernels.ops.scatter2scatter_act(x_src, expert_weights, sorted_expert_idxs, sorted_scattered_idxs, kk,
                                              act_layout, act, b=expert_biases, x_grouped=grouped,
                                              expert_offsets=expert_offsets, alpha=alpha, limit=limit)
        if res is None:     # not a tensor-core case: the two separate kernels
            up = kernels.ops.scatter2scatter(x_src, expert_weights, sorted_expert_idxs, sorted_scattered_idxs, kk,
                                             b=expert_biases, x_grouped=grouped, y_grouped=True,
                                             expert_offsets=expert_offsets)
            F = up.size(1) if act_layout == _act.LAYOUT_PLAIN else up.size(1) // 2
            hidden = torch.empty((up.size(0), F), dtype=up.dtype, device=up.device)
            _act.activation_forward(up, hidden, F, act_layout, act, alpha, limit)
        else:
            up, hidden = res
        ctx.save_for_backward(x, expert_weights, expert_biases, sorted_expert_idxs, sorted_scattered_idxs,
                              expert_offsets, up, x_src if grouped else None)
        ctx.cfg = (k, act_layout, act, alpha, limit)
        return hidden

    @staticmethod
    def backward(ctx, d_hidden):
        (x, expert_weights, expert_biases, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, up,
         x_in_expert_order) = ctx.saved_tensors
        k, act_layout, act, alpha, limit = ctx.cfg
        d_hidden = _rowmajor(d_hidden)
        if d_hidden.dtype != up.dtype:
            d_hidden = d_hidden.to(up.dtype)
        d_up = torch.empty_like(up)
        _act.activation_backward(up, d_hidden, d_up, d_hidden.size(1), act_layout, act, alpha, limit)
        d_input = d_weights = d_biases = None
        if ctx.needs_input_grad[1] or (expert_biases is not None and ctx.needs_input_grad[6]):
            grouped = x_in_expert_order is not None
            d_weights, d_biases = kernels.ops.group_bwd_W(
                DY=d_up, X=x_in_expert_order if grouped else x, expert_offsets=expert_offsets,
                E=expert_weights.size(0), has_bias=expert_biases is not None,
                x_gather_idx=None if grouped else sorted_scattered_idxs, fan_out=1 if grouped else k)
        if ctx.needs_input_grad[0]:
            d_expanded = kernels.ops.scatter2scatter(
                X=d_up, x_grouped=True, W=expert_weights.permute(0, 2, 1), sorted_expert_idxs=sorted_expert_idxs,
                sorted_scattered_idxs=sorted_scattered_idxs, k=1, y_grouped=False, expert_offsets=expert_offsets)
            d_input = d_expanded if k == 1 else kernels.ops.topk_reduce(d_expanded, None, x.size(0), k)
        return (d_input, d_weights, None, None, None, None, d_biases, None, None, None, None)


class ExpertMLP(torch.autograd.Function):
    """Both expert linears, the activation between them and the gate-weighted top-k sum as ONE autograd node, so that
    backward can fuse across the two linears: the input gradient of the down-projection and the activation
    gradient run as one tensor-core launch (`kernels.ops.scatter2scatter_act_bwd`) and the hidden gradient is never
    written. Computes what `ParallelLinear(grouped_out=True)` -> activation -> `ParallelLinear(grouped_in=True,
    gates=...)` compute (scattermoe/mlp.py:33-47, :74-93; scattermoe/parallel_experts.py:27-134), with the same
    saved tensors: the up-projection, the hidden rows and the un-weighted per-slot outputs (the reference's
    `output_expanded`, :45), whose storage backward reuses for the expert-order gradient copy as the reference
    does (:82)."""

    @staticmethod
    def forward(ctx, x, w_up, b_up, w_down, b_down, gates, k, sorted_expert_idxs, sorted_scattered_idxs,
                expert_offsets, act_layout, act, alpha, limit):
        x = _rowmajor(x)
        T = x.size(0)
        x_src, kk, grouped = x, k, False
        if GROUP_INPUT_COPY and x.size(1) % 8 == 0 and x.dtype in (torch.bfloat16, torch.float16):
            x_src, kk, grouped = kernels.ops.group(x, sorted_scattered_idxs, fan_out=k), 1, True
        # the up-projection itself is only kept for backward: without a gradient to compute (inference, torch.no_grad)
        # the fused kernel writes the hidden rows alone
        training = any(ctx.needs_input_grad[:6])
        # Without a bias on the down-projection the gate weighting moves in front of it (the projection is linear): the
        # fused up-projection kernel writes hidden * gate, the per-slot outputs come out weighted and the layer's
        # output is their plain sum. Backward then gets the gate gradient from the same launch that computes the
        # hidden gradient (kernels.ops.scatter2scatter_act_bwd).
        want_gated = (FUSE_GATES and b_down is None and x.dtype in (torch.bfloat16, torch.float16)
                      and kernels.ops.FORCE_PATH != "simt")
        res = kernels.ops.scatter2scatter_act(x_src, w_up, sorted_expert_idxs, sorted_scattered_idxs, kk, act_layout,
                                              act, b=b_up, x_grouped=grouped, expert_offsets=expert_offsets,
                                              alpha=alpha, limit=limit, need_up=training,
                                              row_gates=gates if want_gated else None)
        gated = want_gated and res is not None
        if res is None:     # not a tensor-core case: the two separate kernels
            up = kernels.ops.scatter2scatter(x_src, w_up, sorted_expert_idxs, sorted_scattered_idxs, kk, b=b_up,
                                             x_grouped=grouped, y_grouped=True, expert_offsets=expert_offsets)
            F = up.size(1) if act_layout == _act.LAYOUT_PLAIN else up.size(1) // 2
            hidden = torch.empty((up.size(0), F), dtype=up.dtype, device=up.device)
            _act.activation_forward(up, hidden, F, act_layout, act, alpha, limit)
        else:
            up, hidden = res
        per_slot = kernels.ops.scatter2scatter(hidden, w_down, sorted_expert_idxs, sorted_scattered_idxs, 1, b=b_down,
                                               x_grouped=True, y_grouped=False, expert_offsets=expert_offsets)
        out = kernels.ops.topk_reduce(per_slot, None if gated else gates, T, k)
        ctx.save_for_backward(x, w_up, b_up, w_down, b_down, gates, sorted_expert_idxs, sorted_scattered_idxs,
                              expert_offsets, up, hidden, per_slot, x_src if grouped else None)
        ctx.cfg = (k, act_layout, act, alpha, limit, gated)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (x, w_up, b_up, w_down, b_down, gates, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets, up, hidden,
         per_slot, x_in_expert_order) = ctx.saved_tensors
        k, act_layout, act, alpha, limit, gated = ctx.cfg
        T, E = x.size(0), w_up.size(0)
        need = ctx.needs_input_grad
        grad_out = _rowmajor(grad_out)
        if grad_out.dtype != x.dtype:
            grad_out = grad_out.to(x.dtype)
        d_gates = None
        if need[5] and not gated:
            d_gates = kernels.ops.gate_grad(per_slot, grad_out, T, k).to(gates.dtype)
        d_x = d_w_up = d_b_up = d_w_down = d_b_down = None
        need_up_grad = need[0] or need[1] or (b_up is not None and need[2]) or (gated and need[5])
        if need_up_grad or need[3] or need[4]:
            # the output gradient in expert order (gate-scaled unless the hidden rows carry the gate); written over the
            # per-slot outputs, which nothing reads any more (a traced backward must not write into a tensor saved by
            # forward)
            grouped_grad = kernels.ops.group(grad_out, sorted_scattered_idxs, fan_out=k,
                                             coeff=None if gated else gates.flatten(),
                                             out=None if torch.compiler.is_compiling() else per_slot)
            if need[3] or (b_down is not None and need[4]):
                d_w_down, d_b_down = kernels.ops.group_bwd_W(DY=grouped_grad, X=hidden, expert_offsets=expert_offsets,
                                                             E=E, has_bias=b_down is not None)
            if need_up_grad:
                if gated:
                    d_up, flat = kernels.ops.scatter2scatter_act_bwd(
                        grouped_grad, w_down.permute(0, 2, 1), up, expert_offsets, act_layout, act, alpha, limit,
                        row_gates=gates, sorted_scattered_idxs=sorted_scattered_idxs)
                    if need[5]:
                        d_gates = flat.view(T, k).to(gates.dtype)
                else:
                    d_up = kernels.ops.scatter2scatter_act_bwd(grouped_grad, w_down.permute(0, 2, 1), up, expert_offsets,
                                                               act_layout, act, alpha, limit)
                if need[1] or (b_up is not None and need[2]):
                    grouped = x_in_expert_order is not None
                    d_w_up, d_b_up = kernels.ops.group_bwd_W(
                        DY=d_up, X=x_in_expert_order if grouped else x, expert_offsets=expert_offsets, E=E,
                        has_bias=b_up is not None, x_gather_idx=None if grouped else sorted_scattered_idxs,
                        fan_out=1 if grouped else k)
                if need[0]:
                    d_expanded = kernels.ops.scatter2scatter(
                        X=d_up, x_grouped=True, W=w_up.permute(0, 2, 1), sorted_expert_idxs=sorted_expert_idxs,
                        sorted_scattered_idxs=sorted_scattered_idxs, k=1, y_grouped=False,
                        expert_offsets=expert_offsets)
                    d_x = d_expanded if k == 1 else kernels.ops.topk_reduce(d_expanded, None, T, k)
        return (d_x, d_w_up, d_b_up, d_w_down, d_b_down, d_gates, None, None, None, None, None, None, None, None)


def expert_mlp(inputs, up_weights, down_weights, gates, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
               act_layout, act, up_biases=None, down_biases=None, alpha=1.702, limit=7.0):
    """The whole expert MLP of one MoE layer as one autograd node (an addition to the reference's surface):
    `parallel_linear(grouped_out=True)` -> activation -> `parallel_linear(grouped_in=True, gates=gates)`.
    `up_weights` is (E, in, n_up), `down_weights` (E, hidden, in), any stride order; `gates` (T, k); layout / function
    codes as in `scattermoe_b200.activation`. Input in token order."""
    return ExpertMLP.apply(inputs, up_weights, up_biases, down_weights, down_biases, gates, k, sorted_expert_idxs,
                           sorted_scattered_idxs, expert_offsets, act_layout, act, float(alpha), float(limit))


def parallel_linear_act(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
                        act_layout, act, expert_biases=None, alpha=1.702, limit=7.0):
    """`parallel_linear(..., grouped_out=True)` followed by the activation, as one autograd node (an addition to the
    reference's surface; `scattermoe_b200.activation` has the layout / function codes). Input in token order, 16-bit."""
    return ParallelLinearAct.apply(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs,
                                   expert_offsets, expert_biases, act_layout, act, float(alpha), float(limit))


def parallel_linear(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
                    expert_biases=None, gates=None, grouped_in=False, grouped_out=False):
    """parallel_experts.py:136-146. `expert_weights` is (E, in, out) in any stride order.
    Traceable by torch.compile without graph breaks: every launch below this call is a registered operator
    (`scattermoe_b200::*`) while a trace is being made, and a direct C-ABI call otherwise."""
    return ParallelLinear.apply(inputs, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs,
                                expert_offsets, expert_biases, gates, grouped_in, grouped_out)


class ParallelExperts(nn.Module):
    """parallel_experts.py:148-182: weight (E, out, in) ~ N(0, 0.02), optional bias (E, out) zeros; same
    parameter names and shapes, so reference checkpoints load unchanged."""

    def __init__(self, num_experts, input_size, output_size, bias=False) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, output_size, input_size))
        if bias:
            self.bias = nn.Parameter(torch.empty(num_experts, output_size))
        else:
            self.bias = None
        self.num_experts = num_experts
        self.input_size = input_size
        self.output_size = output_size
        self.reset_parameters()

    def extra_repr(self):
        return 'num_experts={}, input_size={}, output_size={}'.format(
            self.num_experts, self.input_size, self.output_size)

    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, std=0.02)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, inputs, k, sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
                gates=None, grouped_in=False, grouped_out=False):
        return parallel_linear(
            inputs, self.weight.permute(0, 2, 1), k,
            sorted_expert_idxs, sorted_scattered_idxs, expert_offsets,
            expert_biases=self.bias, gates=gates, grouped_in=grouped_in, grouped_out=grouped_out)
