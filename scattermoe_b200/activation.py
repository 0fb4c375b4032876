"""The activation between the two expert linears as one fused pass per direction.

The reference applies `self.activation` with ordinary PyTorch ops (scattermoe/mlp.py:41, :81-87;
scattermoe/utils/replace_moe.py:39-43, :76-83). When the callable is one this library knows (SiLU, GELU, ReLU,
identity) the modules route through `fused_activation` instead: a single kernel forward, a single kernel
backward, nothing kept for backward but the up-projection itself. Any other callable keeps the reference's
behaviour (it is simply called).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import _lib

LAYOUT_PLAIN, LAYOUT_GLU_SECOND, LAYOUT_GLU_FIRST, LAYOUT_GPT_OSS = 0, 1, 2, 3
ACT_SILU, ACT_GELU_ERF, ACT_GELU_TANH, ACT_RELU, ACT_IDENTITY = 0, 1, 2, 3, 4

FUSE = True    # set False to fall back to calling the activation object with PyTorch ops


def _hf_activation_types():
    """Exact Hugging Face activation classes whose forward is one of the functions fused here."""
    try:
        import transformers.activations as hf
    except Exception:
        return {}
    out = {}
    for cls_name, code in (("SiLUActivation", ACT_SILU), ("GELUActivation", ACT_GELU_ERF), ("GELUTanh", ACT_GELU_TANH)):
        cls = getattr(hf, cls_name, None)
        if cls is not None:
            out[cls] = code
    return out


_HF_TYPES = None


def resolve_activation(fn) -> Optional[int]:
    """Activation code for a module / function this library fuses, else None (the callable is then simply called,
    as the reference always does, scattermoe/mlp.py:41, :87). Matching is by identity or EXACT type, never by
    name and never for subclasses: a user class that happens to be called `Swish`, or a subclass overriding
    forward, keeps its own arithmetic."""
    global _HF_TYPES
    if fn is None:
        return None
    Fn = torch.nn.functional
    if fn is Fn.silu:
        return ACT_SILU
    if fn is Fn.gelu:
        return ACT_GELU_ERF
    if fn is Fn.relu:
        return ACT_RELU
    t = type(fn)
    if t is nn.SiLU:
        return ACT_SILU
    if t is nn.GELU:
        return ACT_GELU_TANH if getattr(fn, "approximate", "none") == "tanh" else ACT_GELU_ERF
    if t is nn.ReLU:
        return ACT_RELU
    if t is nn.Identity:
        return ACT_IDENTITY
    if _HF_TYPES is None:
        _HF_TYPES = _hf_activation_types()
    code = _HF_TYPES.get(t)
    if code is not None:
        # these classes pick their implementation in __init__ (`use_gelu_python` and the like): only the default,
        # nn.functional-backed one is the function fused here (the pure-Python variants agree mathematically but
        # the reference would run them as written)
        act = getattr(fn, "act", None)
        if act is None:
            return code
        if act is Fn.gelu and code == ACT_GELU_ERF:
            return code
        import functools
        if (isinstance(act, functools.partial) and act.func is Fn.gelu and act.keywords == {"approximate": "tanh"}
                and not act.args and code == ACT_GELU_TANH):
            return code
        return None
    return None


def _call(backward, up, dh, out, F, layout, act, alpha, limit, rows_dev=None):
    """`rows_dev`: optional device int64 scalar with the live row count (rows beyond it are left untouched)."""
    lib = _lib.load()
    code = _lib.DTYPE_CODE[up.dtype]
    rows = up.size(0)
    rd = 0 if rows_dev is None else rows_dev.data_ptr()
    with torch.cuda.device(up.device):
        if backward:
            rc = lib.smoe_activation_backward(up.data_ptr(), up.stride(0), dh.data_ptr(), dh.stride(0), out.data_ptr(),
                                              out.stride(0), rows, rd, F, layout, act, alpha, limit, code,
                                              _lib.stream_ptr(up.device))
        else:
            rc = lib.smoe_activation_forward(up.data_ptr(), up.stride(0), out.data_ptr(), out.stride(0), rows, rd, F,
                                             layout, act, alpha, limit, code, _lib.stream_ptr(up.device))
    _lib.check(rc, "smoe_activation_backward" if backward else "smoe_activation_forward")


@torch.library.custom_op("scattermoe_b200::activation_forward", mutates_args={"hidden"})
def activation_forward_compileable(up: torch.Tensor, hidden: torch.Tensor, F: int, layout: int, act: int,
                                   alpha: float, limit: float) -> None:
    _call(False, up, None, hidden, F, layout, act, alpha, limit)


@torch.library.custom_op("scattermoe_b200::activation_backward", mutates_args={"d_up"})
def activation_backward_compileable(up: torch.Tensor, d_hidden: torch.Tensor, d_up: torch.Tensor, F: int, layout: int,
                                    act: int, alpha: float, limit: float) -> None:
    _call(True, up, d_hidden, d_up, F, layout, act, alpha, limit)


def activation_forward(up, hidden, F, layout, act, alpha, limit):
    """hidden <- activation(up); the registered operator while torch.compile traces, the direct call otherwise."""
    if torch.compiler.is_compiling():
        activation_forward_compileable(up, hidden, F, layout, act, alpha, limit)
    else:
        _call(False, up, None, hidden, F, layout, act, alpha, limit)


def activation_backward(up, d_hidden, d_up, F, layout, act, alpha, limit):
    """d_up <- d_hidden * activation'(up), same dispatch as `activation_forward`."""
    if torch.compiler.is_compiling():
        activation_backward_compileable(up, d_hidden, d_up, F, layout, act, alpha, limit)
    else:
        _call(True, up, d_hidden, d_up, F, layout, act, alpha, limit)


class FusedActivation(torch.autograd.Function):
    @staticmethod
    def forward(ctx, up: torch.Tensor, layout: int, act: int, alpha: float, limit: float):
        _lib.require_cuda(up, "up")
        if up.stride(-1) != 1:
            up = up.contiguous()
        n_up = up.size(1)
        F = n_up if layout == LAYOUT_PLAIN else n_up // 2
        if layout != LAYOUT_PLAIN and n_up % 2:
            raise AssertionError("gated activation needs an even number of up-projection columns")
        h = torch.empty((up.size(0), F), dtype=up.dtype, device=up.device)
        activation_forward(up, h, F, layout, act, alpha, limit)
        ctx.save_for_backward(up)
        ctx.cfg = (F, layout, act, alpha, limit)
        return h

    @staticmethod
    def backward(ctx, dh: torch.Tensor):
        (up,) = ctx.saved_tensors
        F, layout, act, alpha, limit = ctx.cfg
        if dh.stride(-1) != 1 or dh.dtype != up.dtype:
            dh = dh.to(up.dtype).contiguous()
        d_up = torch.empty_like(up)
        activation_backward(up, dh, d_up, F, layout, act, alpha, limit)
        return d_up, None, None, None, None


def fused_activation(up: torch.Tensor, layout: int, act: int = ACT_SILU, alpha: float = 1.702,
                     limit: float = 7.0) -> torch.Tensor:
    """(rows, n_up) -> (rows, F); see include/scattermoe_b200.h for the layouts."""
    return FusedActivation.apply(up, layout, act, float(alpha), float(limit))
