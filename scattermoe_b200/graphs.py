"""CUDA-graph capture of an MoE layer step.

Every kernel of this package sizes its grid from host-known upper bounds and reads the routing-dependent
quantities (segment offsets, tile counts, live rows) on the device, and nothing on the path synchronises with the
host or allocates outside PyTorch's allocator. A whole forward + backward of a layer is therefore a fixed launch
sequence that can be captured once and replayed for any routing outcome of the same shapes, which removes the
~16 launches and the Python overhead per step that dominate small batches (decode, small micro-batches).

The reference relies on torch.compile for this (README changelog 0.2.0, `@torch.compile` on flatten_sort_count,
scattermoe/parallel_experts.py:14); here it is plain stream capture.
"""
from __future__ import annotations

import torch


def graph_layer(module: torch.nn.Module, sample_args, num_warmup_iters: int = 3):
    """Returns a callable with the module's forward signature whose forward and backward replay CUDA graphs.

    `sample_args`: a tuple of example inputs (same shapes, dtypes and requires_grad flags as the real ones).
    Inputs that do not require grad (the expert indices) are copied into the graph's static buffers on every
    call, so the routing may change freely between calls. The module's parameters are used in place.
    """
    if not all(a.is_cuda for a in sample_args):
        raise RuntimeError("graph_layer needs CUDA tensors: this package has no CPU path")
    return torch.cuda.make_graphed_callables(module, tuple(sample_args), num_warmup_iters=num_warmup_iters,
                                             allow_unused_input=True)
