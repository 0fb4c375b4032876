"""Router fusion: from router logits to gates, expert ids and the routing bookkeeping in one call.

The callers of the reference's `flatten_sort_count` all run the same prologue in PyTorch ops first
(scattermoe/utils/replace_moe.py:67-71 for granite; tests/test_mlp.py:46-51; Hugging Face's gpt-oss router):
softmax over the experts, top-k, optionally a renormalisation, each a kernel with a (T, E) or (T, k) round trip
through HBM, and then the sort. `route_topk` does all of it with three launches: one kernel reads every token's
logits once and writes the selected ids, their gates and the block histograms of the counting sort, then the sort's
scan and scatter kernels run.

    mode "softmax_topk": p = softmax(logits, fp32) over all experts; gates = top-k of p, divided by their sum when
                         `renormalize` (granite, the benchmark configurations) or as they are (the reference test)
    mode "topk_softmax": gates = softmax over the k largest logits (gpt-oss)

Tie rule: larger logit first; equal logits: lower expert id first (torch.topk leaves ties unspecified).
The gates are differentiable with respect to the logits (backward in PyTorch ops on (T, k) / (T, E) tensors).
"""
from __future__ import annotations

import torch

from . import _lib
from .parallel_experts import flatten_sort_count

MODES = {"softmax_topk": 0, "topk_softmax": 1}


def _route_impl(logits: torch.Tensor, k: int, mode: int, renormalize: bool):
    """(gates fp32 (T,k), ids int64 (T,k), lse fp32 (T), sorted_e, sorted_idx, offsets) or None when the request is
    beyond the fused kernel's limits."""
    _lib.require_cuda(logits, "logits")
    T, E = logits.shape
    dev = logits.device
    lib = _lib.load()
    if logits.stride(1) != 1 or logits.dtype not in _lib.DTYPE_CODE:
        logits = logits.contiguous() if logits.dtype in _lib.DTYPE_CODE else logits.float().contiguous()
    R = T * k
    ids = torch.empty((T, k), dtype=torch.int64, device=dev)
    gates = torch.empty((T, k), dtype=torch.float32, device=dev)
    lse = torch.empty((T,), dtype=torch.float32, device=dev)
    sorted_e = torch.empty(R, dtype=torch.int64, device=dev)
    sorted_idx = torch.empty(R, dtype=torch.int64, device=dev)
    offsets = torch.empty(E, dtype=torch.int64, device=dev)
    ws_bytes = lib.smoe_route_topk_workspace_bytes(T, k, E)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.smoe_route_topk(logits.data_ptr(), T, E, logits.stride(0), _lib.DTYPE_CODE[logits.dtype], k, mode,
                                 int(bool(renormalize)), ids.data_ptr(), gates.data_ptr(), lse.data_ptr(),
                                 sorted_e.data_ptr(), sorted_idx.data_ptr(), offsets.data_ptr(), ws.data_ptr(), ws_bytes,
                                 _lib.stream_ptr(dev))
    if rc == _lib.SMOE_ERR_UNSUPPORTED:
        return None
    _lib.check(rc, "smoe_route_topk")
    return gates, ids, lse, sorted_e, sorted_idx, offsets


def _route_unfused(logits: torch.Tensor, k: int, mode: int, renormalize: bool):
    """The same results from separate kernels (expert counts or k beyond the fused kernel's limits)."""
    z = logits.float()
    lse = torch.logsumexp(z, dim=-1)
    top, ids = torch.topk(z, k, dim=-1)
    if mode == MODES["topk_softmax"] or renormalize:
        gates = torch.softmax(top, dim=-1)
    else:
        gates = torch.exp(top - lse.unsqueeze(-1))
    sorted_e, sorted_idx, offsets = flatten_sort_count(ids, logits.size(1))
    return gates, ids, lse, sorted_e, sorted_idx, offsets


@torch.library.custom_op("scattermoe_b200::route_topk", mutates_args={})
def route_topk_compileable(logits: torch.Tensor, k: int, mode: int, renormalize: bool) -> tuple[
        torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    out = _route_impl(logits, k, mode, renormalize)
    return out if out is not None else _route_unfused(logits, k, mode, renormalize)


@route_topk_compileable.register_fake
def _(logits, k, mode, renormalize):
    T, E = logits.shape
    dev = logits.device
    f32, i64 = torch.float32, torch.int64
    return (torch.empty((T, k), dtype=f32, device=dev), torch.empty((T, k), dtype=i64, device=dev),
            torch.empty((T,), dtype=f32, device=dev), torch.empty(T * k, dtype=i64, device=dev),
            torch.empty(T * k, dtype=i64, device=dev), torch.empty(E, dtype=i64, device=dev))


class RouteTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, mode, renormalize):
        with torch.no_grad():
            if torch.compiler.is_compiling():
                out = route_topk_compileable(logits, k, mode, renormalize)
            else:
                out = _route_impl(logits, k, mode, renormalize)
                if out is None:
                    out = _route_unfused(logits, k, mode, renormalize)
        gates, ids, lse, sorted_e, sorted_idx, offsets = out
        softmax_of_selected = mode == MODES["topk_softmax"] or renormalize
        ctx.softmax_of_selected = softmax_of_selected
        ctx.shape = logits.shape
        ctx.in_dtype = logits.dtype
        if softmax_of_selected:
            ctx.save_for_backward(gates, ids)
        else:
            ctx.save_for_backward(gates, ids, logits, lse)
        ctx.mark_non_differentiable(ids, sorted_e, sorted_idx, offsets)
        return gates, ids, sorted_e, sorted_idx, offsets

    @staticmethod
    def backward(ctx, d_gates, *_):
        d_gates = d_gates.float()
        if ctx.softmax_of_selected:
            # gates = softmax over the selected logits: the other logits do not enter
            gates, ids = ctx.saved_tensors
            d_sel = gates * (d_gates - (gates * d_gates).sum(-1, keepdim=True))
            d_logits = torch.zeros(ctx.shape, dtype=torch.float32, device=d_gates.device).scatter_(1, ids, d_sel)
        else:
            # gates_j = p_j of the softmax over all experts: d z_i = sum_j dg_j p_j (delta_ij - p_i)
            gates, ids, logits, lse = ctx.saved_tensors
            p = torch.exp(logits.float() - lse.unsqueeze(-1))
            weighted = d_gates * gates
            d_logits = (-p * weighted.sum(-1, keepdim=True)).scatter_add_(1, ids, weighted)
        return d_logits.to(ctx.in_dtype), None, None, None


def route_topk(logits: torch.Tensor, k: int, mode: str = "softmax_topk", renormalize: bool = True):
    """logits (T, E) -> (gates (T, k) fp32, expert_idxs (T, k) int64, (sorted_expert_idxs, sorted_scattered_idxs,
    expert_offsets)): the router's decision and what `flatten_sort_count(expert_idxs, E)` would return for it."""
    if mode not in MODES:
        raise AssertionError("route_topk: mode must be one of %s" % sorted(MODES))
    if logits.dim() != 2:
        raise AssertionError("route_topk: logits must be (tokens, experts)")
    gates, ids, sorted_e, sorted_idx, offsets = RouteTopK.apply(logits, int(k), MODES[mode], bool(renormalize))
    return gates, ids, (sorted_e, sorted_idx, offsets)
