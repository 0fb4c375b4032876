"""Kernel-level operators, same names and signatures as the reference's scattermoe/kernels/ops.py.

    scatter2scatter  (ops.py:120)   grouped GEMM with fused row gather / scatter
    group_bwd_W      (ops.py:191)   per-expert weight (and bias) gradient
    group            (ops.py:377)   row gather with optional per-row scale
    BLOCK_M, ALLOW_TF32 (ops.py:6-7) module globals read at call time

Every function hands raw device pointers, element strides and the current CUDA stream to the C-ABI library
(include/scattermoe_b200.h). Outputs are allocated here, as in the reference (ops.py:130, :192-195, :384);
the library never allocates. Nothing here computes on the CPU.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib

BLOCK_M = 128        # rows of the expert-sorted slot list per tensor-core tile (ops.py:6)
ALLOW_TF32 = True    # fp32 inputs may use reduced-precision tensor cores (ops.py:7); read at call time
FORCE_PATH = None    # testing hook: None (automatic) | "simt" | "tc"
GATHER_ROWS = False  # testing hook: feed grouped inputs through the cp.async row-gather path instead of TMA


def _flags() -> int:
    f = _lib.FLAG_ALLOW_TF32 if ALLOW_TF32 else 0
    if FORCE_PATH == "simt":
        f |= _lib.FLAG_FORCE_SIMT
    elif FORCE_PATH == "tc":
        f |= _lib.FLAG_FORCE_TC
    if GATHER_ROWS:
        f |= _lib.FLAG_GATHER_ROWS
    return f


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _lib.DTYPE_CODE[t.dtype]
    except KeyError:
        raise RuntimeError("scattermoe_b200: unsupported dtype %s (float32, bfloat16, float16)" % t.dtype)


def _i64(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.int64:
        t = t.to(torch.int64)
    return t if t.is_contiguous() else t.contiguous()


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def last_path_was_tensor_core() -> bool:
    """True if the last GEMM-shaped call made from this thread ran on the tcgen05 kernels."""
    return bool(_lib.load().smoe_last_path_was_tensor_core())


def offsets_from_sorted(sorted_expert_idxs: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Inclusive per-expert end offsets recomputed from the sorted expert ids."""
    _lib.require_cuda(sorted_expert_idxs, "sorted_expert_idxs")
    se = _i64(sorted_expert_idxs)
    out = torch.empty(num_experts, dtype=torch.int64, device=se.device)
    with torch.cuda.device(se.device):
        rc = _lib.load().smoe_offsets_from_sorted(se.data_ptr(), se.numel(), num_experts, out.data_ptr(),
                                                  _lib.stream_ptr(se.device))
    _lib.check(rc, "smoe_offsets_from_sorted")
    return out


# --------------------------------------------------------------------------------------------------
# scatter2scatter
# --------------------------------------------------------------------------------------------------

def _scatter2scatter_impl(output, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped, y_grouped,
                          expert_offsets):
    _lib.require_cuda(X, "X")
    if W.dtype != X.dtype or output.dtype != X.dtype or (b is not None and b.dtype != X.dtype):
        raise RuntimeError("scatter2scatter: X, W, b and the output must share one dtype")
    se, ss = _i64(sorted_expert_idxs), _i64(sorted_scattered_idxs)
    E = W.size(0)
    if expert_offsets is None:
        expert_offsets = offsets_from_sorted(se, E)
    off = _i64(expert_offsets)
    sb = (b.stride(0), b.stride(1)) if b is not None else (0, 0)
    with torch.cuda.device(X.device):
        rc = _lib.load().smoe_scatter2scatter(
            X.data_ptr(), X.size(0), X.stride(0), X.stride(1),
            W.data_ptr(), W.stride(0), W.stride(1), W.stride(2),
            _ptr(b), sb[0], sb[1],
            output.data_ptr(), output.stride(0), output.stride(1),
            se.data_ptr(), ss.data_ptr(), off.data_ptr(),
            se.numel(), X.size(1), output.size(1), E, k,
            int(x_grouped), int(y_grouped), _dtype_code(X), _flags(),
            _lib.status_word(X.device).data_ptr(), _lib.stream_ptr(X.device))
    _lib.check(rc, "smoe_scatter2scatter")


@torch.library.custom_op("scattermoe_b200::scatter2scatter", mutates_args={"output"})
def scatter2scatter_compileable(output: torch.Tensor, W: torch.Tensor, X: torch.Tensor, k: int,
                                sorted_expert_idxs: torch.Tensor, sorted_scattered_idxs: torch.Tensor,
                                b: Optional[torch.Tensor], x_grouped: bool, y_grouped: bool,
                                expert_offsets: Optional[torch.Tensor]) -> None:
    """Traceable form (mirrors scattermoe::scatter2scatter, ops.py:140)."""
    _scatter2scatter_impl(output, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped, y_grouped,
                          expert_offsets)


def scatter2scatter(X, W, sorted_expert_idxs, sorted_scattered_idxs, k, b=None, x_grouped=False, y_grouped=False,
                    out=None, expert_offsets=None):
    """ops.py:120-137. `expert_offsets` is an optional extra: pass it when already known to save the small
    kernel that rebuilds it from `sorted_expert_idxs`."""
    assert sorted_scattered_idxs.size(0) == sorted_expert_idxs.size(0)
    assert sorted_scattered_idxs.size(0) == X.size(0) * k
    y_dim = W.size(-1)
    L_scattered = sorted_expert_idxs.size(0)
    if out is None:
        output = torch.empty((L_scattered, y_dim), device=X.device, dtype=X.dtype)
    else:
        assert out.size(0) == L_scattered and out.size(1) == y_dim
        output = out
    if torch.compiler.is_compiling():
        scatter2scatter_compileable(output, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped,
                                    y_grouped, expert_offsets)
    else:
        _scatter2scatter_impl(output, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped, y_grouped,
                              expert_offsets)
    return output


def _scatter2scatter_act_impl(up, hidden, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped,
                              expert_offsets, act_layout, act, alpha, limit, row_gates=None) -> bool:
    """One launch writing `hidden` (and `up` unless None). False: the request does not fit the tensor-core kernel and
    nothing was launched."""
    _lib.require_cuda(X, "X")
    if FORCE_PATH == "simt" or X.dtype not in (torch.bfloat16, torch.float16) or W.dtype != X.dtype:
        return False
    se, ss = _i64(sorted_expert_idxs), _i64(sorted_scattered_idxs)
    E, N = W.size(0), W.size(-1)
    off = _i64(expert_offsets if expert_offsets is not None else offsets_from_sorted(se, E))
    sb = (b.stride(0), b.stride(1)) if b is not None else (0, 0)
    rg = _flat_gates(row_gates, X.dtype, se.numel())
    with torch.cuda.device(X.device):
        rc = _lib.load().smoe_scatter2scatter_act(
            X.data_ptr(), X.size(0), X.stride(0), X.stride(1),
            W.data_ptr(), W.stride(0), W.stride(1), W.stride(2),
            _ptr(b), sb[0], sb[1],
            _ptr(up), up.stride(0) if up is not None else 0, 1, hidden.data_ptr(), hidden.stride(0),
            se.data_ptr(), ss.data_ptr(), off.data_ptr(),
            se.numel(), X.size(1), N, E, k, int(x_grouped), _dtype_code(X), _flags(),
            act_layout, act, float(alpha), float(limit), _ptr(rg),
            _lib.status_word(X.device).data_ptr(), _lib.stream_ptr(X.device))
    if rc == _lib.SMOE_ERR_UNSUPPORTED:
        return False
    _lib.check(rc, "smoe_scatter2scatter_act")
    return True


def _flat_gates(row_gates, dtype, n):
    """(T, k) gates -> contiguous flat tensor in the compute dtype, indexed by slot."""
    if row_gates is None:
        return None
    g = row_gates.reshape(-1)
    if g.numel() != n:
        raise AssertionError("row_gates has %d entries, %d slots expected" % (g.numel(), n))
    if g.dtype != dtype:
        g = g.to(dtype)
    return g if g.is_contiguous() else g.contiguous()


@torch.library.custom_op("scattermoe_b200::scatter2scatter_act", mutates_args={"up", "hidden"})
def scatter2scatter_act_compileable(up: torch.Tensor, hidden: torch.Tensor, W: torch.Tensor, X: torch.Tensor, k: int,
                                    sorted_expert_idxs: torch.Tensor, sorted_scattered_idxs: torch.Tensor,
                                    b: Optional[torch.Tensor], x_grouped: bool,
                                    expert_offsets: Optional[torch.Tensor], act_layout: int, act: int, alpha: float,
                                    limit: float, row_gates: Optional[torch.Tensor] = None) -> None:
    """Traceable form: always fills both outputs, by the fused kernel when it applies, else by the grouped GEMM
    followed by the activation kernel (a traced graph cannot branch on what the library answers)."""
    if not _scatter2scatter_act_impl(up, hidden, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped,
                                     expert_offsets, act_layout, act, alpha, limit, row_gates):
        from .. import activation as _act
        _scatter2scatter_impl(up, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped, True,
                              expert_offsets)
        _act._call(False, up, None, hidden, hidden.size(1), act_layout, act, alpha, limit)
        if row_gates is not None:
            hidden.mul_(row_gates.reshape(-1).to(hidden.dtype)[sorted_scattered_idxs].unsqueeze(1))


def scatter2scatter_act(X, W, sorted_expert_idxs, sorted_scattered_idxs, k, act_layout, act, b=None, x_grouped=False,
                        expert_offsets=None, alpha=1.702, limit=7.0, need_up=True, row_gates=None):
    """Up-projection into expert order with the activation fused into the kernel's epilogue (the first expert
    linear and the activation of scattermoe/mlp.py:35-41 / :76-87 in one launch). Returns (up, hidden), `up` None
    when `need_up` is False; returns None when the request does not fit the tensor-core kernel (the caller then
    uses `scatter2scatter` and the activation kernel; while torch.compile traces, that choice is made inside the
    registered operator and the result is never None). Layout / function codes: scattermoe_b200.activation.
    `row_gates` ((T, k), optional): `hidden` rows are multiplied by the gate of their slot (`up` is not)."""
    assert sorted_scattered_idxs.size(0) == sorted_expert_idxs.size(0)
    assert sorted_scattered_idxs.size(0) == X.size(0) * k
    R, N = sorted_expert_idxs.size(0), W.size(-1)
    F = N if act_layout == 0 else N // 2
    if torch.compiler.is_compiling():
        up = torch.empty((R, N), device=X.device, dtype=X.dtype)
        hidden = torch.empty((R, F), device=X.device, dtype=X.dtype)
        scatter2scatter_act_compileable(up, hidden, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped,
                                        expert_offsets, act_layout, act, float(alpha), float(limit), row_gates)
        return up, hidden
    up = torch.empty((R, N), device=X.device, dtype=X.dtype) if need_up else None
    hidden = torch.empty((R, F), device=X.device, dtype=X.dtype)
    if not _scatter2scatter_act_impl(up, hidden, W, X, k, sorted_expert_idxs, sorted_scattered_idxs, b, x_grouped,
                                     expert_offsets, act_layout, act, alpha, limit, row_gates):
        return None
    return up, hidden


def _scatter2scatter_act_bwd_impl(d_up, DY, W, up, expert_offsets, act_layout, act, alpha, limit, row_gates=None,
                                  sorted_scattered_idxs=None, partials=None) -> bool:
    """One launch writing `d_up` = activation gradient of (DY @ W) with respect to the saved up-projection `up`
    (and, with gates, the gate gradient's partial sums into `partials`). False: the request does not fit the
    tensor-core kernel and nothing was launched."""
    _lib.require_cuda(DY, "DY")
    if FORCE_PATH == "simt" or DY.dtype not in (torch.bfloat16, torch.float16) or W.dtype != DY.dtype:
        return False
    if up.dtype != DY.dtype or up.stride(1) != 1 or d_up.stride(1) != 1 or d_up.shape != up.shape:
        return False
    off = _i64(expert_offsets)
    rg = _flat_gates(row_gates, DY.dtype, DY.size(0))
    ss = _i64(sorted_scattered_idxs) if rg is not None else None
    with torch.cuda.device(DY.device):
        rc = _lib.load().smoe_scatter2scatter_act_bwd(
            DY.data_ptr(), DY.stride(0), DY.stride(1),
            W.data_ptr(), W.stride(0), W.stride(1), W.stride(2),
            up.data_ptr(), up.stride(0), d_up.data_ptr(), d_up.stride(0),
            off.data_ptr(), DY.size(0), DY.size(1), W.size(-1), W.size(0), _dtype_code(DY), _flags(),
            act_layout, act, float(alpha), float(limit), _ptr(rg), _ptr(ss), _ptr(partials if rg is not None else None),
            _lib.status_word(DY.device).data_ptr(), _lib.stream_ptr(DY.device))
    if rc == _lib.SMOE_ERR_UNSUPPORTED:
        return False
    _lib.check(rc, "smoe_scatter2scatter_act_bwd")
    return True


def _partial_lines(F: int) -> int:
    return 2 * ((F + 255) // 256)


def _gate_grad_from_partials(partials, sorted_scattered_idxs, dtype):
    R = partials.size(1)
    d_gates = torch.empty(R, dtype=dtype, device=partials.device)
    ss = _i64(sorted_scattered_idxs)
    with torch.cuda.device(partials.device):
        rc = _lib.load().smoe_gate_grad_from_partials(partials.data_ptr(), partials.size(0), R, ss.data_ptr(),
                                                      d_gates.data_ptr(), _lib.DTYPE_CODE[dtype],
                                                      _lib.stream_ptr(partials.device))
    _lib.check(rc, "smoe_gate_grad_from_partials")
    return d_gates


@torch.library.custom_op("scattermoe_b200::scatter2scatter_act_bwd", mutates_args={"d_up"})
def scatter2scatter_act_bwd_compileable(d_up: torch.Tensor, DY: torch.Tensor, W: torch.Tensor, up: torch.Tensor,
                                        expert_offsets: torch.Tensor, act_layout: int, act: int, alpha: float,
                                        limit: float) -> None:
    """Traceable form: always fills `d_up`, by the fused kernel when it applies, else by the grouped GEMM followed by
    the activation-gradient kernel."""
    _scatter2scatter_act_bwd_fill(d_up, DY, W, up, expert_offsets, act_layout, act, alpha, limit)


@torch.library.custom_op("scattermoe_b200::scatter2scatter_act_bwd_gated", mutates_args={"d_up", "d_gates"})
def scatter2scatter_act_bwd_gated_compileable(d_up: torch.Tensor, d_gates: torch.Tensor, DY: torch.Tensor, W: torch.Tensor,
                                              up: torch.Tensor, expert_offsets: torch.Tensor, act_layout: int, act: int,
                                              alpha: float, limit: float, row_gates: torch.Tensor,
                                              sorted_scattered_idxs: torch.Tensor) -> None:
    """Traceable form of the variant that takes the un-weighted output gradient and the gates: fills `d_up` and
    `d_gates` (flat by slot)."""
    _scatter2scatter_act_bwd_fill(d_up, DY, W, up, expert_offsets, act_layout, act, alpha, limit, row_gates,
                                  sorted_scattered_idxs, d_gates)


def _scatter2scatter_act_bwd_fill(d_up, DY, W, up, expert_offsets, act_layout, act, alpha, limit, row_gates=None,
                                  sorted_scattered_idxs=None, d_gates=None):
    F = W.size(-1)
    R = DY.size(0)
    partials = None
    if row_gates is not None:
        partials = torch.empty((_partial_lines(F), R), dtype=torch.float32, device=DY.device)
    if _scatter2scatter_act_bwd_impl(d_up, DY, W, up, expert_offsets, act_layout, act, alpha, limit, row_gates,
                                     sorted_scattered_idxs, partials):
        if row_gates is not None:
            d_gates.copy_(_gate_grad_from_partials(partials, sorted_scattered_idxs, d_gates.dtype))
        return
    # the two separate kernels (CUDA cores for fp32 / unaligned shapes)
    from .. import activation as _act
    d_hidden = torch.empty((R, F), device=DY.device, dtype=DY.dtype)
    # rows are in expert order on both sides; the CUDA-core kernel still reads each row's expert id
    rows = torch.arange(R, device=DY.device, dtype=torch.int64)
    sorted_e = torch.searchsorted(_i64(expert_offsets), rows, right=True)
    _scatter2scatter_impl(d_hidden, W, DY, 1, sorted_e, rows, None, True, True, expert_offsets)
    if row_gates is not None:
        # gate gradient <hidden (un-weighted), d_hidden (un-weighted)> per row, then the gate on the hidden gradient
        hidden = torch.empty_like(d_hidden)
        _act._call(False, up, None, hidden, F, act_layout, act, alpha, limit)
        slots = _i64(sorted_scattered_idxs)
        d_gates[slots] = (hidden.float() * d_hidden.float()).sum(-1).to(d_gates.dtype)
        d_hidden = d_hidden * row_gates.reshape(-1).to(d_hidden.dtype)[slots].unsqueeze(1)
    _act._call(True, up, d_hidden, d_up, F, act_layout, act, alpha, limit)


def scatter2scatter_act_bwd(DY, W, up, expert_offsets, act_layout, act, alpha=1.702, limit=7.0, row_gates=None,
                            sorted_scattered_idxs=None):
    """Gradient of the up-projection `up` (rows, n_up) given the gradient `DY` (rows, K) of the down-projection's
    OUTPUT, rows in expert order: d_up = activation'(up) applied to DY @ W, with W the (E, K, F) transposed view of
    the down-projection weight. One tensor-core launch whose epilogue applies the activation gradient (the
    autograd of scattermoe/mlp.py:41 / :81-87 fused into the grouped GEMM of scattermoe/parallel_experts.py:110-116);
    the (rows, F) hidden gradient is not materialised. Falls back to the two separate kernels when the request does
    not fit the tensor-core kernel.

    With `row_gates` ((T, k)) and `sorted_scattered_idxs`, DY is the UN-weighted output gradient: the hidden gradient
    is scaled by each row's gate inside the epilogue, which also yields the gate gradient (the row dot product of
    scattermoe/parallel_experts.py:79, taken on the hidden side of the down-projection). Returns (d_up, d_gates)
    then, d_gates flat by slot in the dtype of DY."""
    d_up = torch.empty_like(up)
    d_gates = None
    if row_gates is not None:
        d_gates = torch.empty(DY.size(0), dtype=DY.dtype, device=DY.device)
    if torch.compiler.is_compiling():
        if row_gates is None:
            scatter2scatter_act_bwd_compileable(d_up, DY, W, up, expert_offsets, act_layout, act, float(alpha),
                                                float(limit))
        else:
            scatter2scatter_act_bwd_gated_compileable(d_up, d_gates, DY, W, up, expert_offsets, act_layout, act,
                                                      float(alpha), float(limit), row_gates, sorted_scattered_idxs)
    else:
        _scatter2scatter_act_bwd_fill(d_up, DY, W, up, expert_offsets, act_layout, act, alpha, limit, row_gates,
                                      sorted_scattered_idxs, d_gates)
    return d_up if row_gates is None else (d_up, d_gates)


def scatter2scatter_to_peers(X, W, expert_offsets, return_addr, peer_ptrs, peer_stride_rows, peer_rows, rank,
                             world) -> bool:
    """Grouped GEMM of the local experts whose epilogue stores every result row straight into its home rank's buffer
    over NVLink (expert parallelism, the return direction): `scatter2scatter(X, W, ..., x_grouped=True,
    y_grouped=True)` followed by `smoe_ep_return`, as one tensor-core launch without the local result buffer. X is the
    owner's expert-grouped (capacity, K) buffer, W (E_local, K, N), `return_addr` the (capacity,) int64 (rank, row)
    records written by `smoe_ep_dispatch`, `peer_ptrs` the ctypes table of the ranks' (peer_rows, peer_stride_rows)
    buffers. False: the request does not fit the tensor-core kernel and nothing was launched (the caller runs the two
    separate calls). No counterpart in the reference, which has no multi-GPU code."""
    _lib.require_cuda(X, "X")
    if FORCE_PATH == "simt" or X.dtype not in (torch.bfloat16, torch.float16) or W.dtype != X.dtype:
        return False
    off, ret = _i64(expert_offsets), _i64(return_addr)
    if ret.numel() < X.size(0):
        raise AssertionError("return_addr has %d entries for %d rows" % (ret.numel(), X.size(0)))
    with torch.cuda.device(X.device):
        rc = _lib.load().smoe_scatter2scatter_to_peers(
            X.data_ptr(), X.size(0), X.stride(0), X.stride(1), W.data_ptr(), W.stride(0), W.stride(1), W.stride(2),
            off.data_ptr(), ret.data_ptr(), peer_ptrs, int(peer_stride_rows), int(peer_rows), int(world), int(rank),
            X.size(1), W.size(-1), W.size(0), _dtype_code(X), _flags(), _lib.status_word(X.device).data_ptr(),
            _lib.stream_ptr(X.device))
    if rc == _lib.SMOE_ERR_UNSUPPORTED:
        return False
    _lib.check(rc, "smoe_scatter2scatter_to_peers")
    return True


# --------------------------------------------------------------------------------------------------
# group_bwd_W
# --------------------------------------------------------------------------------------------------

def _group_bwd_w_impl(E, DWt, Db, DY, X, expert_offsets, x_gather_idx, fan_out):
    _lib.require_cuda(DY, "DY")
    DW = DWt.permute(0, 2, 1)
    if X.dtype != DY.dtype or DW.dtype != DY.dtype:
        raise RuntimeError("group_bwd_W: DY, X and DW must share one dtype")
    off = _i64(expert_offsets)
    gi = _i64(x_gather_idx) if x_gather_idx is not None else None
    sdb = (Db.stride(0), Db.stride(1)) if Db is not None else (0, 0)
    with torch.cuda.device(DY.device):
        rc = _lib.load().smoe_group_bwd_w(
            DY.data_ptr(), DY.stride(0), DY.stride(1),
            X.data_ptr(), X.size(0), X.stride(0), X.stride(1),
            off.data_ptr(), _ptr(gi), fan_out,
            DW.data_ptr(), DW.stride(0), DW.stride(1), DW.stride(2),
            _ptr(Db), sdb[0], sdb[1],
            DY.size(0), X.size(1), DY.size(1), E, _dtype_code(DY), _flags(),
            _lib.status_word(DY.device).data_ptr(), _lib.stream_ptr(DY.device))
    _lib.check(rc, "smoe_group_bwd_w")


@torch.library.custom_op("scattermoe_b200::groupXtY", mutates_args={"DWt", "Db"})
def groupXtY_compileable(E: int, DWt: torch.Tensor, Db: Optional[torch.Tensor], DY: torch.Tensor, X: torch.Tensor,
                         expert_offsets: torch.Tensor, x_gather_idx: Optional[torch.Tensor], fan_out: int) -> None:
    """Traceable form (mirrors scattermoe::groupXtY, ops.py:202; Db is declared as mutated here). `DWt` is the
    (E, N, K) buffer whose (E, K, N) view is the gradient: the operator mutates a base tensor, not a view."""
    _group_bwd_w_impl(E, DWt, Db, DY, X, expert_offsets, x_gather_idx, fan_out)


def group_bwd_W(DY, X, expert_offsets, E, has_bias=False, x_gather_idx=None, fan_out=1):
    """ops.py:191-199. Returns (DW as the (E,K,N) view of an (E,N,K) buffer, Db or None).

    Extension: with `x_gather_idx` (the sorted slot indices) X may be the un-grouped (T, K) input; row m then
    reads X[x_gather_idx[m] // fan_out], which makes the reference's `group(x)` copy unnecessary.
    The kernel writes every element (zeros for experts without rows), so the buffers are not pre-zeroed.
    """
    if x_gather_idx is None:
        assert X.size(0) == DY.size(0)
    else:
        assert x_gather_idx.size(0) == DY.size(0) and X.size(0) * fan_out == DY.size(0)
    DWt = torch.empty((E, DY.size(-1), X.size(-1)), device=DY.device, dtype=DY.dtype)
    DW = DWt.permute(0, 2, 1)
    Db = torch.empty((E, DY.size(-1)), device=DY.device, dtype=DY.dtype) if has_bias else None
    if torch.compiler.is_compiling():
        groupXtY_compileable(E, DWt, Db, DY, X, expert_offsets, x_gather_idx, fan_out)
    else:
        _group_bwd_w_impl(E, DWt, Db, DY, X, expert_offsets, x_gather_idx, fan_out)
    return DW, Db


# --------------------------------------------------------------------------------------------------
# group
# --------------------------------------------------------------------------------------------------

def _group_impl(A, K, N, Y, coeff, has_coeff, fan_out, sorted_expert_idxs):
    _lib.require_cuda(A, "A")
    if Y.dtype != A.dtype:
        raise RuntimeError("group: A and the output must share one dtype")
    idx = _i64(sorted_expert_idxs)
    c = None
    if has_coeff:
        c = coeff if (coeff.dtype == A.dtype and coeff.is_contiguous()) else coeff.to(A.dtype).contiguous()
    with torch.cuda.device(A.device):
        rc = _lib.load().smoe_group(A.data_ptr(), A.size(0), A.stride(0), A.stride(1), idx.data_ptr(), _ptr(c),
                                    fan_out, Y.data_ptr(), Y.stride(0), Y.stride(1), N, K, _dtype_code(A),
                                    _lib.stream_ptr(A.device))
    _lib.check(rc, "smoe_group")


@torch.library.custom_op("scattermoe_b200::group", mutates_args={"Y"})
def group_compileable(A: torch.Tensor, K: int, N: int, Y: torch.Tensor, coeff: Optional[torch.Tensor],
                      has_coeff: bool, fan_out: int, sorted_expert_idxs: torch.Tensor) -> None:
    """Traceable form (mirrors scattermoe::group, ops.py:389)."""
    _group_impl(A, K, N, Y, coeff, has_coeff, fan_out, sorted_expert_idxs)


def group(A, sorted_expert_idxs, coeff=None, fan_out=1, out=None):
    """ops.py:377-386. The index argument keeps the reference's name although every caller passes the
    sorted slot indices (parallel_experts.py:92, :99)."""
    N = sorted_expert_idxs.size(0)
    K = A.size(1)
    assert A.size(0) * fan_out == N
    if out is not None:
        Y = out
    else:
        Y = torch.empty((N, K), dtype=A.dtype, device=A.device)
    if torch.compiler.is_compiling():
        group_compileable(A, K, N, Y, coeff, coeff is not None, fan_out, sorted_expert_idxs)
    else:
        _group_impl(A, K, N, Y, coeff, coeff is not None, fan_out, sorted_expert_idxs)
    return Y


# --------------------------------------------------------------------------------------------------
# top-k reductions (torch ops in the reference, parallel_experts.py:44-46, :79, :123)
# --------------------------------------------------------------------------------------------------

def _topk_reduce_impl(expanded: torch.Tensor, gates: Optional[torch.Tensor], T: int, k: int) -> torch.Tensor:
    _lib.require_cuda(expanded, "expanded")
    assert expanded.size(0) == T * k
    if expanded.stride(1) != 1:
        expanded = expanded.contiguous()
    N = expanded.size(1)
    out = torch.empty((T, N), dtype=expanded.dtype, device=expanded.device)
    g = None
    if gates is not None:
        assert gates.size(0) == T and gates.size(1) == k
        g = gates if gates.dtype == expanded.dtype else gates.to(expanded.dtype)
    sg = (g.stride(0), g.stride(1)) if g is not None else (0, 0)
    with torch.cuda.device(expanded.device):
        rc = _lib.load().smoe_topk_reduce(expanded.data_ptr(), expanded.stride(0), _ptr(g), sg[0], sg[1],
                                          out.data_ptr(), out.stride(0), T, k, N, _dtype_code(expanded),
                                          _lib.stream_ptr(expanded.device))
    _lib.check(rc, "smoe_topk_reduce")
    return out


@torch.library.custom_op("scattermoe_b200::topk_reduce", mutates_args={})
def topk_reduce_compileable(expanded: torch.Tensor, gates: Optional[torch.Tensor], T: int, k: int) -> torch.Tensor:
    return _topk_reduce_impl(expanded, gates, T, k)


@topk_reduce_compileable.register_fake
def _(expanded, gates, T, k):
    return torch.empty((T, expanded.size(1)), dtype=expanded.dtype, device=expanded.device)


def topk_reduce(expanded: torch.Tensor, gates: Optional[torch.Tensor], T: int, k: int) -> torch.Tensor:
    """out[t] = sum_j gates[t, j] * expanded[t*k + j]  (gates None: plain sum). `expanded` is (T*k, N)."""
    if torch.compiler.is_compiling():
        return topk_reduce_compileable(expanded, gates, T, k)
    return _topk_reduce_impl(expanded, gates, T, k)


def _gate_grad_impl(expanded: torch.Tensor, grad_out: torch.Tensor, T: int, k: int) -> torch.Tensor:
    _lib.require_cuda(expanded, "expanded")
    assert expanded.size(0) == T * k and grad_out.size(0) == T
    if expanded.stride(1) != 1:
        expanded = expanded.contiguous()
    if grad_out.stride(1) != 1 or grad_out.dtype != expanded.dtype:
        grad_out = grad_out.to(expanded.dtype).contiguous()
    dg = torch.empty((T, k), dtype=expanded.dtype, device=expanded.device)
    with torch.cuda.device(expanded.device):
        rc = _lib.load().smoe_gate_grad(expanded.data_ptr(), expanded.stride(0), grad_out.data_ptr(),
                                        grad_out.stride(0), dg.data_ptr(), dg.stride(0), dg.stride(1), T, k,
                                        expanded.size(1), _dtype_code(expanded), _lib.stream_ptr(expanded.device))
    _lib.check(rc, "smoe_gate_grad")
    return dg


@torch.library.custom_op("scattermoe_b200::gate_grad", mutates_args={})
def gate_grad_compileable(expanded: torch.Tensor, grad_out: torch.Tensor, T: int, k: int) -> torch.Tensor:
    return _gate_grad_impl(expanded, grad_out, T, k)


@gate_grad_compileable.register_fake
def _(expanded, grad_out, T, k):
    return torch.empty((T, k), dtype=expanded.dtype, device=expanded.device)


def gate_grad(expanded: torch.Tensor, grad_out: torch.Tensor, T: int, k: int) -> torch.Tensor:
    """d_gates[t, j] = <expanded[t*k + j], grad_out[t]>, in the dtype of `expanded`."""
    if torch.compiler.is_compiling():
        return gate_grad_compileable(expanded, grad_out, T, k)
    return _gate_grad_impl(expanded, grad_out, T, k)
