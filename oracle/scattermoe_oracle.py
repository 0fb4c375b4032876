"""CPU oracle for the ScatterMoE `ParallelLinear` hot path.

THIS FILE IS TEST INFRASTRUCTURE. It is a plain CPU (torch, fp32/fp64) restatement of what
the reference computes, written as per-expert dense loops. Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it; the product package never
does and has no CPU fallback.

Parity status: PINNED. `tests/golden/make_golden.py` runs the reference package itself
(its Triton kernels executed by the Triton interpreter on CPU) on seeded inputs and stores
the inputs and outputs; `tests/test_oracle.py` checks every function below against those
stored vectors.

Each function cites the reference file:line it restates (paths inside the reference
project).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

# --------------------------------------------------------------------------------------
# routing bookkeeping
# --------------------------------------------------------------------------------------


def flatten_sort_count(expert_idxs: torch.Tensor, num_experts: int):
    """scattermoe/parallel_experts.py:14-21.

    Flatten the (T, k) expert ids, sort them ascending, return (sorted ids, the flat slot
    index `t*k+j` of every sorted entry, inclusive cumulative per-expert counts). The
    reference calls torch.sort without stable=True; the oracle fixes the tie order as the
    stable one (ascending slot index inside one expert), which is the only order that is
    well defined.
    """
    flat = expert_idxs.reshape(-1).to(torch.int64)
    sorted_expert_idxs, sorted_scattered_idxs = torch.sort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    expert_offsets = counts.cumsum(-1)
    return sorted_expert_idxs, sorted_scattered_idxs, expert_offsets


def offsets_from_sorted(sorted_expert_idxs: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Inclusive end offsets recovered from the sorted ids alone (what the reference kernel
    does implicitly by masking rows per expert, scattermoe/kernels/ops.py:81-91)."""
    counts = torch.bincount(sorted_expert_idxs.to(torch.int64), minlength=num_experts)
    return counts.cumsum(-1)


def _segments(expert_offsets: torch.Tensor):
    ends = expert_offsets.tolist()
    start = 0
    for e, end in enumerate(ends):
        yield e, start, end
        start = end


# --------------------------------------------------------------------------------------
# kernels
# --------------------------------------------------------------------------------------


def scatter2scatter(X, W, sorted_expert_idxs, sorted_scattered_idxs, k, b=None,
                    x_grouped=False, y_grouped=False, acc_dtype=torch.float32):
    """scattermoe/kernels/ops.py:120-137 (wrapper) and :55-118 (kernel).

    Row m of the expert-sorted slot list is multiplied by its expert's (K, N) matrix.
    Input row: m itself if x_grouped else slot // k (ops.py:93-96). Output row: m if
    y_grouped else the slot index (ops.py:113-116). Bias of the row's expert is added
    (ops.py:109-111). Accumulation in fp32 (ops.py:180), result in X's dtype (ops.py:130).
    """
    R = sorted_expert_idxs.numel()
    assert sorted_scattered_idxs.numel() == R and R == X.size(0) * k
    N = W.size(-1)
    E = W.size(0)
    Y = torch.zeros((R, N), dtype=X.dtype)
    offsets = offsets_from_sorted(sorted_expert_idxs, E)
    for e, s, t in _segments(offsets):
        if t == s:
            continue
        slots = sorted_scattered_idxs[s:t]
        rows_in = torch.arange(s, t) if x_grouped else torch.div(slots, k, rounding_mode="floor")
        acc = X[rows_in].to(acc_dtype) @ W[e].to(acc_dtype)
        if b is not None:
            acc = acc + b[e].to(acc_dtype)
        rows_out = torch.arange(s, t) if y_grouped else slots
        Y[rows_out] = acc.to(X.dtype)
    return Y


def group(A, sorted_scattered_idxs, coeff=None, fan_out=1):
    """scattermoe/kernels/ops.py:377-386 and :417-457.

    Y[n, :] = A[idx[n] // fan_out, :] * coeff[idx[n]].
    """
    idx = sorted_scattered_idxs.to(torch.int64)
    assert A.size(0) * fan_out == idx.numel()
    Y = A[torch.div(idx, fan_out, rounding_mode="floor")]
    if coeff is not None:
        Y = (Y.float() * coeff.reshape(-1)[idx].float()[:, None]).to(A.dtype)
    return Y.clone()


def group_bwd_W(DY, X, expert_offsets, E, has_bias=False, acc_dtype=torch.float32):
    """scattermoe/kernels/ops.py:191-199 and :247-366.

    Per expert e over its contiguous row segment of the grouped X and DY:
    DW[e] (K, N) = X_e^T DY_e, Db[e] = column sums of DY_e; experts with no rows give
    exact zeros (ops.py:192-195, :279). The buffer is (E, N, K) contiguous and the
    returned DW is its (E, K, N) permuted view (ops.py:192-193); dtype of DY.
    """
    N, K = DY.size(-1), X.size(-1)
    DWt = torch.zeros((E, N, K), dtype=DY.dtype)
    Db = torch.zeros((E, N), dtype=DY.dtype) if has_bias else None
    for e, s, t in _segments(expert_offsets):
        if t == s:
            continue
        dy = DY[s:t].to(acc_dtype)
        DWt[e] = (dy.t() @ X[s:t].to(acc_dtype)).to(DY.dtype)
        if has_bias:
            Db[e] = dy.sum(0).to(DY.dtype)
    return DWt.permute(0, 2, 1), Db


# --------------------------------------------------------------------------------------
# autograd orchestration (forward and backward of one expert linear)
# --------------------------------------------------------------------------------------


def parallel_linear_forward(x, expert_weights, k, sorted_expert_idxs, sorted_scattered_idxs,
                            expert_offsets, expert_biases=None, gates=None,
                            grouped_in=False, grouped_out=False):
    """scattermoe/parallel_experts.py:27-62. Returns (output, output_expanded)."""
    out = scatter2scatter(x, expert_weights, sorted_expert_idxs, sorted_scattered_idxs, k,
                          b=expert_biases, x_grouped=grouped_in, y_grouped=grouped_out)
    if gates is None:
        return out, None
    expanded = out.view(gates.size(0), gates.size(1), out.size(-1))
    y = (gates.float().unsqueeze(1) @ expanded.float()).squeeze(1).to(out.dtype)   # :44-46
    return y, expanded


def parallel_linear_backward(grad_out, x, expert_weights, k, sorted_expert_idxs,
                             sorted_scattered_idxs, expert_offsets, expert_biases=None,
                             gates=None, output_expanded=None, grouped_in=False,
                             grouped_out=False):
    """scattermoe/parallel_experts.py:64-134.

    Returns (d_input, d_weights, d_biases, d_gates).
    """
    E = expert_weights.size(0)
    if gates is not None:
        d_gates = (output_expanded.float() @ grad_out.float().unsqueeze(-1)).squeeze(-1).to(gates.dtype)  # :79
        gates_flat, gate_fan = gates.reshape(-1), gates.size(1)
    else:
        d_gates, gates_flat, gate_fan = None, None, 1
    if grouped_out:
        grouped_grad_out = grad_out                                                  # :89-90
    else:
        grouped_grad_out = group(grad_out, sorted_scattered_idxs, coeff=gates_flat, fan_out=gate_fan)  # :92-94
    grouped_x = x if grouped_in else group(x, sorted_scattered_idxs, fan_out=k)      # :95-99
    d_weights, d_biases = group_bwd_W(grouped_grad_out, grouped_x, expert_offsets, E,
                                      has_bias=expert_biases is not None)            # :102-107
    d_expanded = scatter2scatter(grouped_grad_out, expert_weights.permute(0, 2, 1),
                                 sorted_expert_idxs, sorted_scattered_idxs, 1,
                                 x_grouped=True, y_grouped=grouped_in)               # :110-118
    if k == 1:
        d_input = d_expanded
    else:
        d_input = d_expanded.view(x.size(0), k, d_expanded.size(-1)).float().sum(-2).to(x.dtype)  # :120-123
    return d_input, d_weights, d_biases, d_gates


# --------------------------------------------------------------------------------------
# single-token path
# --------------------------------------------------------------------------------------

def single2scatter(X, W, expert_idxs):
    """scattermoe/kernels/single.py:41-60 (_single2scatter :6-39): one token routed to k experts.
    Y[j] = X[j if X has k rows else 0] @ W[expert_idxs[0, j]], fp32 accumulation, output in X's dtype."""
    k = expert_idxs.size(1)
    assert X.size(0) == k or X.size(0) == 1
    rows = []
    for j in range(k):
        x = X[j if X.size(0) == k else 0].to(torch.float32)
        rows.append(x @ W[int(expert_idxs[0, j])].to(torch.float32))
    return torch.stack(rows).to(X.dtype)


# --------------------------------------------------------------------------------------
# activations placed between the two expert linears
# --------------------------------------------------------------------------------------


def route_topk(logits, k, mode="softmax_topk", renormalize=True):
    """The router prologue that every caller of flatten_sort_count runs first, restated: fp32 softmax over the
    experts, top-k, division by the sum of the selected probabilities (scattermoe/utils/replace_moe.py:67-71, the
    granite patch; `renormalize=False` is the reference test's router, tests/test_mlp.py:46-51), or, for
    mode "topk_softmax", top-k of the logits followed by a softmax over the selected ones (the gpt-oss router whose
    outputs scattermoe/utils/replace_moe.py:22-27 consumes). Returns (gates (T, k) fp32, expert ids (T, k) int64)."""
    z = logits.float()
    if mode == "topk_softmax":
        top, ids = torch.topk(z, k, dim=-1)
        return torch.softmax(top, dim=-1), ids
    p = torch.softmax(z, dim=-1)
    g, ids = torch.topk(p, k, dim=-1)
    if renormalize:
        g = g / g.sum(-1, keepdim=True)
    return g, ids


def act_gelu(h):
    """nn.GELU() default (erf form), as used by tests/test_mlp.py:55."""
    return torch.nn.functional.gelu(h)


def act_glu_second_half(h2, act=torch.nn.functional.silu):
    """scattermoe/mlp.py:81-87: `h, gates = chunk(2)`; `act(gates) * h`."""
    h, g = h2.chunk(2, dim=-1)
    return act(g) * h


def act_glu_first_half(h2, act=torch.nn.functional.silu):
    """scattermoe/utils/replace_moe.py:76-83: `gates, h = chunk(2)`; `act(gates) * h`."""
    g, h = h2.chunk(2, dim=-1)
    return act(g) * h


def act_gpt_oss(gate_up, alpha=1.702, limit=7.0):
    """scattermoe/utils/replace_moe.py:39-43: interleaved columns, clamped SwiGLU."""
    gate, up = gate_up[..., ::2], gate_up[..., 1::2]
    gate = gate.clamp(min=None, max=limit)
    up = up.clamp(min=-limit, max=limit)
    return (up + 1) * (gate * torch.sigmoid(gate * alpha))


# --------------------------------------------------------------------------------------
# whole MoE MLP, dense per-expert loop with autograd: the independent second oracle
# --------------------------------------------------------------------------------------


def dense_moe_mlp(x, expert_p, expert_idxs, w1, w2, b1=None, b2=None, activation=act_gelu,
                  compute_dtype=None):
    """Same maths as `dumb_forward` in tests/test_mlp.py:10-26, one matmul per expert
    instead of one per (token, slot). `w1` is (E, d_in, n1) and `w2` (E, f, d_out) in
    logical (in, out) orientation; `activation` maps (rows, n1) -> (rows, f).
    Differentiable with torch autograd.
    """
    T, k = expert_idxs.shape
    E = w1.size(0)
    cd = compute_dtype or x.dtype
    y = torch.zeros((T, w2.size(-1)), dtype=cd)
    flat_e = expert_idxs.reshape(-1)
    tok = torch.arange(T).repeat_interleave(k)
    flat_p = expert_p.reshape(-1)
    for e in range(E):
        sel = (flat_e == e).nonzero().squeeze(-1)
        if sel.numel() == 0:
            continue
        t_idx = tok[sel]
        h = x[t_idx].to(cd) @ w1[e].to(cd)
        if b1 is not None:
            h = h + b1[e].to(cd)
        h = activation(h)
        o = h @ w2[e].to(cd)
        if b2 is not None:
            o = o + b2[e].to(cd)
        y = y.index_add(0, t_idx, o * flat_p[sel].to(cd)[:, None])
    return y


def moe_mlp_forward_backward(x, expert_p, expert_idxs, w1, w2, b1, b2, activation, grad_out,
                             compute_dtype=torch.float32):
    """Forward and gradients of `dense_moe_mlp` w.r.t. x, expert_p, w1, w2 (and biases).
    Returns dict of tensors in `compute_dtype`."""
    leaves = {"x": x, "expert_p": expert_p, "w1": w1, "w2": w2}
    if b1 is not None:
        leaves["b1"] = b1
    if b2 is not None:
        leaves["b2"] = b2
    leaves = {n: t.detach().to(compute_dtype).requires_grad_() for n, t in leaves.items()}
    y = dense_moe_mlp(leaves["x"], leaves["expert_p"], expert_idxs, leaves["w1"], leaves["w2"],
                      leaves.get("b1"), leaves.get("b2"), activation, compute_dtype)
    grads = torch.autograd.grad(y, list(leaves.values()), grad_out.to(compute_dtype))
    out = {"y": y.detach()}
    for n, g in zip(leaves.keys(), grads):
        out["d_" + n] = g
    return out


# --------------------------------------------------------------------------------------
# seeded synthetic workloads (shapes and value distributions of the benchmark configs)
# --------------------------------------------------------------------------------------

CONFIGS = {
    # name: T, d_model, d_ffn, E, top_k, kind, bias, dtype
    "tiny_fp32_gelu": dict(T=256, d=128, F=256, E=8, k=2, kind="mlp_gelu", bias=False, dtype="float32"),
    "mixtral_8x7b": dict(T=16384, d=4096, F=14336, E=8, k=2, kind="glu_silu", bias=False, dtype="bfloat16"),
    "gpt_oss_20b": dict(T=8192, d=2880, F=2880, E=32, k=4, kind="gpt_oss", bias=True, dtype="bfloat16"),
    "granite_zipf": dict(T=32768, d=1536, F=512, E=64, k=8, kind="glu_silu", bias=False, dtype="bfloat16"),
    "qwen3_moe_ep": dict(T=65536, d=2048, F=768, E=128, k=8, kind="glu_silu", bias=False, dtype="bfloat16"),
}


def make_routing(cfg_name: str, T: int, E: int, k: int, seed: int = 0):
    """Router outputs for one config: (expert_p (T,k) fp32, expert_idxs (T,k) int64)."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if cfg_name == "granite_zipf":
        pop = torch.arange(1, E + 1, dtype=torch.float32) ** -1.2
        pop = pop / pop.sum()
        perm = torch.randperm(E, generator=g)
        logits = logits + torch.log(pop)[perm]
    if cfg_name == "gpt_oss_20b":
        top, idx = torch.topk(logits, k, dim=-1)
        p = torch.softmax(top, dim=-1)
    else:
        p_full = torch.softmax(logits, dim=-1)
        p, idx = torch.topk(p_full, k, dim=-1)
        p = p / p.sum(-1, keepdim=True)
    return p, idx


class DenseLoopBench:
    """One layer of a benchmark config with fp32 weights, for timing the dense per-expert loop on the host
    cores (the CPU baseline). Weights and inputs are built once; `step()` runs forward (+ backward)."""

    def __init__(self, cfg_name: str, T_sample: int, threads: Optional[int] = None, seed: int = 0):
        cfg = CONFIGS[cfg_name]
        if threads:
            torch.set_num_threads(threads)
        self.threads = torch.get_num_threads()
        d, F, E, k = cfg["d"], cfg["F"], cfg["E"], cfg["k"]
        n1 = F if cfg["kind"] == "mlp_gelu" else 2 * F
        g = torch.Generator().manual_seed(seed)
        dt = torch.float32
        self.x = torch.randn(T_sample, d, generator=g, dtype=dt)
        self.w1 = torch.empty(E, d, n1, dtype=dt).normal_(0, 0.02, generator=g)
        self.w2 = torch.empty(E, F, d, dtype=dt).normal_(0, 0.02, generator=g)
        self.b1 = torch.randn(E, n1, generator=g, dtype=dt) * 0.02 if cfg["bias"] else None
        self.b2 = torch.randn(E, d, generator=g, dtype=dt) * 0.02 if cfg["bias"] else None
        self.p, self.idx = make_routing(cfg_name, T_sample, E, k, seed)
        self.act = {"mlp_gelu": act_gelu, "glu_silu": act_glu_second_half, "gpt_oss": act_gpt_oss}[cfg["kind"]]
        self.go = torch.randn(T_sample, d, generator=g, dtype=dt)

    def step(self, backward: bool = True) -> float:
        import time
        t0 = time.perf_counter()
        if backward:
            moe_mlp_forward_backward(self.x, self.p, self.idx, self.w1, self.w2, self.b1, self.b2, self.act, self.go,
                                     compute_dtype=torch.float32)
        else:
            with torch.no_grad():
                dense_moe_mlp(self.x, self.p, self.idx, self.w1, self.w2, self.b1, self.b2, self.act, torch.float32)
        return time.perf_counter() - t0
