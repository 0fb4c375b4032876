"""Single-token expert matvec, same name and signature as the reference's scattermoe/kernels/single.py:41-59.

The reference does not import this module from `kernels/__init__.py` and nothing in the reference calls it; it is
kept here the same way (import it explicitly: `from scattermoe_b200.kernels import single`).
"""
import torch

from .. import _lib


def single2scatter(X, W, expert_idxs):
    """Y[j] = X[j or 0] @ W[expert_idxs[0, j]] for the k experts of one token (single.py:41-59).
    X: (1, K) or (k, K); W: (E, K, N) in any stride order; expert_idxs: (1, k). fp32 accumulation."""
    _lib.require_cuda(X, "X")
    E, xdim, ydim = W.size()
    k = expert_idxs.size(1)
    assert X.size(0) == k or X.size(0) == 1
    if W.dtype != X.dtype:
        raise RuntimeError("single2scatter: X and W must share one dtype")
    Y = torch.empty((k, ydim), device=X.device, dtype=X.dtype)
    idx = expert_idxs.reshape(-1)
    if idx.dtype != torch.int64 or not idx.is_contiguous():
        idx = idx.to(torch.int64).contiguous()
    with torch.cuda.device(X.device):
        rc = _lib.load().smoe_single2scatter(X.data_ptr(), X.size(0), X.stride(0), X.stride(1), W.data_ptr(),
                                             W.stride(0), W.stride(1), W.stride(2), Y.data_ptr(), Y.stride(0),
                                             Y.stride(1), idx.data_ptr(), k, xdim, ydim, E, _lib.DTYPE_CODE[X.dtype],
                                             _lib.stream_ptr(X.device))
    _lib.check(rc, "smoe_single2scatter")
    return Y
