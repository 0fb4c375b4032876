"""Kernel-level parity on the GPU through the C ABI: golden vectors from the reference, and the oracle on
seeded inputs, for both the tensor-core (tcgen05) and the CUDA-core paths."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import scattermoe_oracle as oracle  # noqa: E402
from util import as_dtype, assert_close, golden_names, load_golden  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    import scattermoe_b200 as sm
    from scattermoe_b200.kernels import ops
    ops.FORCE_PATH = None
    yield
    ops.FORCE_PATH = None
    sm.check_device_status()      # no kernel may have given up on a wait


def _dev(t):
    return None if t is None else t.cuda()


@pytest.mark.parametrize("path", ["auto", "simt"])
@pytest.mark.parametrize("name", golden_names("s2s_"))
def test_scatter2scatter_golden(name, path):
    from scattermoe_b200.kernels import ops
    g = load_golden(name)
    X, b = as_dtype(g, g["X"]), as_dtype(g, g.get("b"))
    W = as_dtype(g, g["W"])
    if not g["w_n_contiguous"]:
        W = W.permute(0, 2, 1).contiguous().permute(0, 2, 1)     # K-contiguous storage, as the reference ran it
    ops.FORCE_PATH = None if path == "auto" else path
    Y = ops.scatter2scatter(_dev(X), _dev(W), _dev(g["sorted_expert_idxs"]), _dev(g["sorted_scattered_idxs"]), g["k"],
                            b=_dev(b), x_grouped=g["x_grouped"], y_grouped=g["y_grouped"])
    assert_close(name, Y, g["Y"], g["bf16"])
    with_off = ops.scatter2scatter(_dev(X), _dev(W), _dev(g["sorted_expert_idxs"]), _dev(g["sorted_scattered_idxs"]),
                                   g["k"], b=_dev(b), x_grouped=g["x_grouped"], y_grouped=g["y_grouped"],
                                   expert_offsets=_dev(g["expert_offsets"]))
    assert torch.equal(with_off, Y)


@pytest.mark.parametrize("name", golden_names("group_"))
def test_group_golden(name):
    from scattermoe_b200.kernels import ops
    g = load_golden(name)
    A, c = as_dtype(g, g["A"]), as_dtype(g, g.get("coeff"))
    Y = ops.group(_dev(A), _dev(g["sorted_scattered_idxs"]), coeff=_dev(c), fan_out=g["k"])
    assert_close(name, Y, g["Y"], g["bf16"])
    out = torch.empty_like(Y)
    assert ops.group(_dev(A), _dev(g["sorted_scattered_idxs"]), coeff=_dev(c), fan_out=g["k"], out=out) is out
    assert torch.equal(out, Y)


@pytest.mark.parametrize("path", ["auto", "simt"])
@pytest.mark.parametrize("name", golden_names("gbw_"))
def test_group_bwd_w_golden(name, path):
    from scattermoe_b200.kernels import ops
    g = load_golden(name)
    ops.FORCE_PATH = None if path == "auto" else path
    DW, Db = ops.group_bwd_W(_dev(as_dtype(g, g["DY"])), _dev(as_dtype(g, g["X"])), _dev(g["expert_offsets"]), g["E"],
                             has_bias="Db" in g)
    assert DW.shape == g["DW"].shape and DW.stride(1) == 1, "(E,K,N) view of an (E,N,K) buffer"
    assert_close(name + ".DW", DW, g["DW"], g["bf16"])
    if "Db" in g:
        assert_close(name + ".Db", Db, g["Db"], g["bf16"])
    counts = torch.bincount(g["expert_idxs"].flatten(), minlength=g["E"])
    assert bool((DW.cpu()[counts == 0] == 0).all())


def _routing(T, E, k, seed, skew=False):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if skew:
        logits[:, : max(1, E // 3)] -= 30.0
        logits[:, -1] += 2.0
    p = torch.softmax(logits, -1)
    w, idx = torch.topk(p, k)
    return w / w.sum(-1, keepdim=True), idx, g


TC_SHAPES = [
    # T, E, k, K, N
    (300, 4, 2, 64, 128),
    (1000, 8, 2, 256, 512),
    (513, 8, 3, 320, 264),      # K and N tails (not multiples of 64 / 256)
    (64, 16, 4, 128, 2880 // 4),  # many small experts, N = 720
    (2048, 8, 2, 1024, 384),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("w_layout", ["k_contig", "n_contig"])
@pytest.mark.parametrize("mode", [(False, True), (True, False), (True, True), (False, False)])
@pytest.mark.parametrize("shape", TC_SHAPES)
def test_scatter2scatter_tensor_core_vs_oracle(shape, mode, w_layout, dtype):
    from scattermoe_b200.kernels import ops
    T, E, k, K, N = shape
    x_grouped, y_grouped = mode
    _, idx, g = _routing(T, E, k, seed=T + K + N, skew=(T % 2 == 1))
    se, ss, off = oracle.flatten_sort_count(idx, E)
    kk = 1 if x_grouped else k
    X = torch.randn(T * k if x_grouped else T, K, generator=g).to(dtype)
    if w_layout == "n_contig":
        W = (torch.randn(E, K, N, generator=g) * 0.05).to(dtype)
    else:
        W = (torch.randn(E, N, K, generator=g) * 0.05).to(dtype).permute(0, 2, 1)
    b = (torch.randn(E, N, generator=g) * 0.1).to(dtype) if (T + K) % 3 else None
    ops.FORCE_PATH = "tc"
    Y = ops.scatter2scatter(_dev(X), _dev(W), _dev(se), _dev(ss), kk, b=_dev(b), x_grouped=x_grouped,
                            y_grouped=y_grouped, expert_offsets=_dev(off))
    assert ops.last_path_was_tensor_core()
    want = oracle.scatter2scatter(X.float(), W.float(), se, ss, kk, b=None if b is None else b.float(),
                                  x_grouped=x_grouped, y_grouped=y_grouped)
    assert_close("Y", Y, want, True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("gathered", [False, True])
@pytest.mark.parametrize("shape", [(300, 4, 2, 64, 128), (1000, 8, 2, 256, 512), (513, 8, 3, 320, 264),
                                   (40, 16, 4, 136, 72), (2048, 8, 2, 384, 1024)])
def test_group_bwd_w_tensor_core_vs_oracle(shape, gathered, dtype):
    from scattermoe_b200.kernels import ops
    T, E, k, K, N = shape
    _, idx, g = _routing(T, E, k, seed=T + K + N + 1, skew=True)
    se, ss, off = oracle.flatten_sort_count(idx, E)
    DY = torch.randn(T * k, N, generator=g).to(dtype)
    if gathered:
        X = torch.randn(T, K, generator=g).to(dtype)
        Xg = oracle.group(X, ss, fan_out=k)
    else:
        Xg = X = torch.randn(T * k, K, generator=g).to(dtype)
    ops.FORCE_PATH = "tc"
    DW, Db = ops.group_bwd_W(_dev(DY), _dev(X), _dev(off), E, has_bias=True,
                             x_gather_idx=_dev(ss) if gathered else None, fan_out=k if gathered else 1)
    assert ops.last_path_was_tensor_core()
    wDW, wDb = oracle.group_bwd_W(DY.float(), Xg.float(), off, E, has_bias=True)
    scale = max(1.0, float((T * k / E) ** 0.5))     # sums over ~R/E rows of unit-variance products
    assert_close("DW", DW.float().cpu() / scale, wDW / scale, True)
    assert_close("Db", Db.float().cpu() / scale, wDb / scale, True)
    counts = torch.bincount(idx.flatten(), minlength=E)
    assert bool((DW.cpu()[counts == 0] == 0).all()) and bool((Db.cpu()[counts == 0] == 0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,k,N", [(1, 2, 8), (33, 3, 100), (200, 4, 512), (64, 1, 72)])
def test_topk_reduce_and_gate_grad(T, k, N, dtype):
    from scattermoe_b200.kernels import ops
    g = torch.Generator().manual_seed(T + k + N)
    Yx = torch.randn(T * k, N, generator=g).to(dtype)
    gates = torch.rand(T, k, generator=g).to(dtype)
    go = torch.randn(T, N, generator=g).to(dtype)
    bf16 = dtype == torch.bfloat16
    out = ops.topk_reduce(_dev(Yx), _dev(gates), T, k)
    want = (gates.float().unsqueeze(1) @ Yx.float().view(T, k, N)).squeeze(1)
    assert_close("reduce", out, want, bf16)
    out = ops.topk_reduce(_dev(Yx), None, T, k)
    assert_close("sum", out, Yx.float().view(T, k, N).sum(1), bf16)
    dg = ops.gate_grad(_dev(Yx), _dev(go), T, k)
    want = (Yx.float().view(T, k, N) @ go.float().unsqueeze(-1)).squeeze(-1)
    if bf16:
        torch.testing.assert_close(dg.float().cpu(), want, rtol=2e-2, atol=2e-2 * N ** 0.5)
    else:
        torch.testing.assert_close(dg.cpu(), want, rtol=1e-4, atol=1e-4)


def test_shape_contract_violations_raise_assertion_errors():
    from scattermoe_b200.kernels import ops
    idx = torch.zeros(6, dtype=torch.int64, device="cuda")
    X = torch.zeros(4, 8, device="cuda")
    W = torch.zeros(2, 8, 8, device="cuda")
    with pytest.raises(AssertionError):
        ops.scatter2scatter(X, W, idx, idx, 2)          # 6 != 4 * 2   (ops.py:125)
    with pytest.raises(AssertionError):
        ops.group(X, idx, fan_out=1)                    # ops.py:380
    with pytest.raises(AssertionError):
        ops.scatter2scatter(X, W, idx[:4], idx[:4], 1, out=torch.zeros(3, 8, device="cuda"))   # ops.py:132


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,F", [(5, 8), (33, 133), (100, 256), (7, 20)])
@pytest.mark.parametrize("layout,act", [("plain", "gelu"), ("plain", "silu"), ("glu_second", "silu"),
                                        ("glu_second", "gelu"), ("glu_first", "silu"), ("gpt_oss", None)])
def test_fused_activation_forward_and_backward(rows, F, layout, act, dtype):
    """One-pass activation kernels against the PyTorch formulas the reference uses (mlp.py:41, :81-87;
    replace_moe.py:39-43, :76-83), forward and autograd backward."""
    from scattermoe_b200 import activation as A
    g = torch.Generator().manual_seed(rows * 31 + F)
    n_up = F if layout == "plain" else 2 * F
    up = (torch.randn(rows, n_up, generator=g) * 3).to(dtype)     # wide enough to hit the gpt-oss clamps at +-7
    dh = torch.randn(rows, F, generator=g).to(dtype)
    ref_in = up.float().requires_grad_()
    fn = {"gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu, None: None}[act]
    if layout == "plain":
        ref = fn(ref_in)
    elif layout == "glu_second":
        ref = oracle.act_glu_second_half(ref_in, fn)
    elif layout == "glu_first":
        ref = oracle.act_glu_first_half(ref_in, fn)
    else:
        ref = oracle.act_gpt_oss(ref_in)
    (ref_grad,) = torch.autograd.grad(ref, ref_in, dh.float())
    code = {"gelu": A.ACT_GELU_ERF, "silu": A.ACT_SILU, None: A.ACT_SILU}[act]
    lay = {"plain": A.LAYOUT_PLAIN, "glu_second": A.LAYOUT_GLU_SECOND, "glu_first": A.LAYOUT_GLU_FIRST,
           "gpt_oss": A.LAYOUT_GPT_OSS}[layout]
    x = up.cuda().requires_grad_()
    h = A.fused_activation(x, lay, code, 1.702, 7.0)
    (gx,) = torch.autograd.grad(h, x, dh.cuda())
    bf16 = dtype == torch.bfloat16
    if bf16:
        torch.testing.assert_close(h.float().cpu(), ref.detach(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(gx.float().cpu(), ref_grad, rtol=2e-2, atol=4e-2)
    else:
        torch.testing.assert_close(h.cpu(), ref.detach(), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(gx.cpu(), ref_grad, rtol=1e-5, atol=2e-5)


def test_activation_resolution():
    from torch import nn
    from scattermoe_b200 import activation as A
    assert A.resolve_activation(nn.SiLU()) == A.ACT_SILU
    assert A.resolve_activation(nn.GELU()) == A.ACT_GELU_ERF
    assert A.resolve_activation(nn.GELU(approximate="tanh")) == A.ACT_GELU_TANH
    assert A.resolve_activation(nn.ReLU()) == A.ACT_RELU
    assert A.resolve_activation(nn.Identity()) == A.ACT_IDENTITY
    assert A.resolve_activation(nn.Tanh()) is None and A.resolve_activation(lambda t: t) is None
    from transformers.activations import ACT2FN, GELUActivation
    assert A.resolve_activation(ACT2FN["silu"]) == A.ACT_SILU
    assert A.resolve_activation(ACT2FN["gelu"]) == A.ACT_GELU_ERF
    assert A.resolve_activation(ACT2FN["gelu_pytorch_tanh"]) == A.ACT_GELU_TANH
    assert A.resolve_activation(GELUActivation(use_gelu_python=True)) is None
    assert A.resolve_activation(ACT2FN["gelu_new"]) is None

    class Swish(nn.Module):                 # same name as a fused function, different arithmetic: must not be fused
        def __init__(self, beta):
            super().__init__()
            self.beta = beta

        def forward(self, t):
            return t * torch.sigmoid(self.beta * t)

    class MySiLU(nn.SiLU):
        def forward(self, t):
            return 2 * super().forward(t)
    assert A.resolve_activation(Swish(1.5)) is None and A.resolve_activation(MySiLU()) is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["n_contig", "k_contig"])
@pytest.mark.parametrize("K,N,k,x_rows", [(128, 256, 2, 1), (256, 128, 4, 4), (100, 72, 3, 1), (1000, 520, 2, 2)])
def test_single2scatter(K, N, k, x_rows, layout, dtype):
    """Decode matvec against the formula of the reference kernel (kernels/single.py:5-39)."""
    from scattermoe_b200.kernels import single
    E = 6
    g = torch.Generator().manual_seed(K + N + k)
    X = torch.randn(x_rows, K, generator=g).to(dtype)
    W = (torch.randn(E, K, N, generator=g) * 0.1).to(dtype)
    idx = torch.randint(0, E, (1, k), generator=g)
    Wd = W.cuda() if layout == "n_contig" else W.permute(0, 2, 1).contiguous().cuda().permute(0, 2, 1)
    Y = single.single2scatter(X.cuda(), Wd, idx.cuda())
    want = torch.stack([X[j if x_rows > 1 else 0].float() @ W[idx[0, j]].float() for j in range(k)])
    assert Y.shape == (k, N) and Y.dtype == dtype
    if dtype == torch.bfloat16:
        torch.testing.assert_close(Y.float().cpu(), want, rtol=2e-2, atol=2e-2)
    else:
        torch.testing.assert_close(Y.cpu(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("w_layout", ["k_contig", "n_contig"])
@pytest.mark.parametrize("layout,act,bias", [("plain", "gelu", True), ("glu_second", "silu", False), ("glu_first", "silu", True),
                                             ("gpt_oss", None, True)])
@pytest.mark.parametrize("T,E,k,K,F", [(300, 4, 2, 64, 136), (513, 8, 3, 320, 200), (1000, 8, 2, 256, 384)])
def test_fused_up_projection_and_activation(T, E, k, K, F, layout, act, bias, w_layout):
    """The activation fused into the epilogue of the tensor-core grouped GEMM (one launch) against the oracle's
    scatter2scatter followed by the PyTorch formulas; both outputs (up-projection and hidden) are checked."""
    from scattermoe_b200 import activation as A
    from scattermoe_b200.kernels import ops
    dtype = torch.bfloat16
    N = F if layout == "plain" else 2 * F
    _, idx, g = _routing(T, E, k, seed=T + K + F, skew=True)
    se, ss, off = oracle.flatten_sort_count(idx, E)
    X = torch.randn(T, K, generator=g).to(dtype)
    if w_layout == "n_contig":
        W = (torch.randn(E, K, N, generator=g) * 0.1).to(dtype)
    else:
        W = (torch.randn(E, N, K, generator=g) * 0.1).to(dtype).permute(0, 2, 1)
    b = (torch.randn(E, N, generator=g) * 0.5).to(dtype) if bias else None
    lay = {"plain": A.LAYOUT_PLAIN, "glu_second": A.LAYOUT_GLU_SECOND, "glu_first": A.LAYOUT_GLU_FIRST,
           "gpt_oss": A.LAYOUT_GPT_OSS}[layout]
    code = {"gelu": A.ACT_GELU_ERF, "silu": A.ACT_SILU, None: A.ACT_SILU}[act]
    res = ops.scatter2scatter_act(_dev(X), _dev(W), _dev(se), _dev(ss), k, lay, code, b=_dev(b), expert_offsets=_dev(off))
    assert res is not None, "this shape must take the fused tensor-core kernel"
    up, hidden = res
    want_up = oracle.scatter2scatter(X.float(), W.float(), se, ss, k, b=None if b is None else b.float(), y_grouped=True)
    fn = {"gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu, None: None}[act]
    if layout == "plain":
        want_h = fn(want_up)
    elif layout == "glu_second":
        want_h = oracle.act_glu_second_half(want_up, fn)
    elif layout == "glu_first":
        want_h = oracle.act_glu_first_half(want_up, fn)
    else:
        want_h = oracle.act_gpt_oss(want_up)
    assert_close("up", up, want_up, True)
    assert_close("hidden", hidden, want_h, True, atol_scale=max(1.0, want_h.abs().max().item() / 4))
    # without the up-projection output (inference)
    res2 = ops.scatter2scatter_act(_dev(X), _dev(W), _dev(se), _dev(ss), k, lay, code, b=_dev(b), expert_offsets=_dev(off),
                                   need_up=False)
    assert res2[0] is None and torch.equal(res2[1], hidden)


def test_fused_up_projection_declines_what_it_cannot_do():
    from scattermoe_b200 import activation as A
    from scattermoe_b200.kernels import ops
    idx = torch.zeros(8, dtype=torch.int64, device="cuda")
    se, ss = idx, torch.arange(8, device="cuda")
    X32 = torch.zeros(8, 64, device="cuda")
    assert ops.scatter2scatter_act(X32, torch.zeros(1, 64, 256, device="cuda"), se, ss, 1, A.LAYOUT_PLAIN, A.ACT_SILU) is None
    Xb = X32.bfloat16()
    assert ops.scatter2scatter_act(Xb, torch.zeros(1, 64, 64, device="cuda", dtype=torch.bfloat16), se, ss, 1,
                                   A.LAYOUT_PLAIN, A.ACT_SILU) is None          # N <= 128


def _act_reference(layout, act, up):
    fn = {"gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu, None: None}[act]
    if layout == "plain":
        return fn(up)
    if layout == "glu_second":
        return oracle.act_glu_second_half(up, fn)
    if layout == "glu_first":
        return oracle.act_glu_first_half(up, fn)
    return oracle.act_gpt_oss(up)


def _act_codes(layout, act):
    from scattermoe_b200 import activation as A
    lay = {"plain": A.LAYOUT_PLAIN, "glu_second": A.LAYOUT_GLU_SECOND, "glu_first": A.LAYOUT_GLU_FIRST,
           "gpt_oss": A.LAYOUT_GPT_OSS}[layout]
    return lay, {"gelu": A.ACT_GELU_ERF, "silu": A.ACT_SILU, None: A.ACT_SILU}[act]


@pytest.mark.parametrize("w_layout", ["k_contig", "n_contig"])
@pytest.mark.parametrize("layout,act", [("plain", "gelu"), ("glu_second", "silu"), ("glu_first", "gelu"), ("gpt_oss", None)])
@pytest.mark.parametrize("T,E,k,K,F", [(300, 4, 2, 64, 136), (300, 4, 2, 64, 144), (513, 8, 3, 320, 200), (1000, 8, 2, 256, 384),
                                       (2048, 4, 2, 128, 1024)])
def test_fused_input_gradient_and_activation_gradient(T, E, k, K, F, layout, act, w_layout):
    """The activation gradient fused into the epilogue of the down-projection's input-gradient GEMM (one launch,
    the hidden gradient never stored) against the oracle's scatter2scatter followed by PyTorch autograd of the
    reference's activation formulas (mlp.py:41, :81-87; replace_moe.py:39-43, :76-83)."""
    from scattermoe_b200.kernels import ops
    dtype = torch.bfloat16
    n_up = F if layout == "plain" else 2 * F
    _, idx, g = _routing(T, E, k, seed=T + K + F + 5, skew=True)
    se, ss, off = oracle.flatten_sort_count(idx, E)
    R = T * k
    DY = torch.randn(R, K, generator=g).to(dtype)                  # gradient of the down-projection's output, grouped
    up = (torch.randn(R, n_up, generator=g) * 2.5).to(dtype)       # wide enough to reach the gpt-oss clamps
    if w_layout == "n_contig":
        W = (torch.randn(E, K, F, generator=g) * 0.1).to(dtype)
    else:
        W = (torch.randn(E, F, K, generator=g) * 0.1).to(dtype).permute(0, 2, 1)
    lay, code = _act_codes(layout, act)
    ops.FORCE_PATH = "tc"
    from scattermoe_b200 import _lib
    d_up = torch.full((R, n_up), float("nan"), dtype=dtype, device="cuda")
    assert ops._scatter2scatter_act_bwd_impl(d_up, _dev(DY), _dev(W), _dev(up), _dev(off), lay, code, 1.702, 7.0), \
        "this shape must take the fused tensor-core kernel: " + _lib.last_error()
    d_hidden = oracle.scatter2scatter(DY.float(), W.float(), se, ss, 1, x_grouped=True, y_grouped=True)
    ref_in = up.float().requires_grad_()
    (want,) = torch.autograd.grad(_act_reference(layout, act, ref_in), ref_in, d_hidden)
    assert not bool(torch.isnan(d_up).any()), "every element of the gradient must be written"
    assert_close("d_up", d_up, want, True, atol_scale=max(1.0, want.abs().max().item() / 4))
    # the public wrapper gives the same bits, and the split path (grouped GEMM, then the activation-gradient kernel)
    # agrees within the rounding of the stored hidden gradient
    again = ops.scatter2scatter_act_bwd(_dev(DY), _dev(W), _dev(up), _dev(off), lay, code)
    assert torch.equal(again, d_up)
    ops.FORCE_PATH = "simt"
    split = ops.scatter2scatter_act_bwd(_dev(DY), _dev(W), _dev(up), _dev(off), lay, code)
    assert_close("d_up (split path)", split, want, True, atol_scale=max(1.0, want.abs().max().item() / 4))


def _zipf_routing(T, E, k, seed):
    """Skewed load: a few experts take most rows, some take none (the shape of the granite-style config)."""
    g = torch.Generator().manual_seed(seed)
    pop = torch.arange(1, E + 1, dtype=torch.float32) ** -1.2
    logits = torch.randn(T, E, generator=g) + torch.log(pop / pop.sum())[torch.randperm(E, generator=g)]
    return torch.topk(logits, k).indices, g


LONG_WALKS = [
    # T, E, k, K, N: every CTA of the persistent kernels walks >= 4 tiles, so tensor-memory buffers and the
    # shared-memory ring are reused many times inside one launch (as at benchmark sizes)
    (65536, 8, 2, 64, 256, False),      # 1024 row tiles x 1 column tile
    (32768, 8, 4, 128, 512, False),     # 1024 x 2
    (16384, 64, 8, 128, 256, True),     # zipf: ragged, tiny and empty experts among 1024+ row tiles
]


@pytest.mark.parametrize("mode", [(False, True), (True, False), (True, True), (False, False)])
@pytest.mark.parametrize("T,E,k,K,N,zipf", LONG_WALKS)
def test_scatter2scatter_many_tiles_per_cta(T, E, k, K, N, zipf, mode):
    from scattermoe_b200.kernels import ops
    x_grouped, y_grouped = mode
    if zipf:
        idx, g = _zipf_routing(T, E, k, seed=T + E)
    else:
        _, idx, g = _routing(T, E, k, seed=T + E + K)
    se, ss, off = oracle.flatten_sort_count(idx, E)
    kk = 1 if x_grouped else k
    X = torch.randn(T * k if x_grouped else T, K, generator=g).bfloat16()
    W = (torch.randn(E, N, K, generator=g) * 0.05).bfloat16().permute(0, 2, 1)
    b = (torch.randn(E, N, generator=g) * 0.1).bfloat16()
    ops.FORCE_PATH = "tc"
    Y = ops.scatter2scatter(_dev(X), _dev(W), _dev(se), _dev(ss), kk, b=_dev(b), x_grouped=x_grouped,
                            y_grouped=y_grouped, expert_offsets=_dev(off))
    assert ops.last_path_was_tensor_core()
    want = oracle.scatter2scatter(X.float(), W.float(), se, ss, kk, b=b.float(), x_grouped=x_grouped, y_grouped=y_grouped)
    assert_close("Y", Y, want, True)


@pytest.mark.parametrize("layout,act", [("glu_second", "silu"), ("gpt_oss", None), ("plain", "gelu")])
@pytest.mark.parametrize("T,E,k,K,N,zipf", LONG_WALKS)
def test_fused_epilogues_many_tiles_per_cta(T, E, k, K, N, zipf, layout, act):
    """Both fused epilogue families (activation after the up-projection; activation gradient after the
    down-projection's input gradient) on launches in which a CTA walks many tiles."""
    from scattermoe_b200.kernels import ops
    if zipf:
        idx, g = _zipf_routing(T, E, k, seed=T + E + 1)
    else:
        _, idx, g = _routing(T, E, k, seed=T + E + K + 1)
    se, ss, off = oracle.flatten_sort_count(idx, E)
    R = T * k
    lay, code = _act_codes(layout, act)
    n_up = N if layout == "plain" else 2 * N            # N plays the part of the hidden width F here
    X = torch.randn(T, K, generator=g).bfloat16()
    W1 = (torch.randn(E, n_up, K, generator=g) * 0.1).bfloat16().permute(0, 2, 1)
    res = ops.scatter2scatter_act(_dev(X), _dev(W1), _dev(se), _dev(ss), k, lay, code, expert_offsets=_dev(off))
    assert res is not None
    up, hidden = res
    want_up = oracle.scatter2scatter(X.float(), W1.float(), se, ss, k, y_grouped=True)
    assert_close("up", up, want_up, True)
    want_h = _act_reference(layout, act, want_up)
    assert_close("hidden", hidden, want_h, True, atol_scale=max(1.0, want_h.abs().max().item() / 4))
    DY = torch.randn(R, K, generator=g).bfloat16()
    W2t = (torch.randn(E, K, N, generator=g) * 0.1).bfloat16()      # (E, K, F): transposed view of the down-projection
    ops.FORCE_PATH = "tc"
    d_up = torch.full((R, n_up), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert ops._scatter2scatter_act_bwd_impl(d_up, _dev(DY), _dev(W2t), up, _dev(off), lay, code, 1.702, 7.0)
    d_hidden = oracle.scatter2scatter(DY.float(), W2t.float(), se, ss, 1, x_grouped=True, y_grouped=True)
    ref_in = up.float().cpu().requires_grad_()
    (want,) = torch.autograd.grad(_act_reference(layout, act, ref_in), ref_in, d_hidden)
    assert_close("d_up", d_up, want, True, atol_scale=max(1.0, want.abs().max().item() / 4))


@pytest.mark.parametrize("gathered", [False, True])
@pytest.mark.parametrize("T,E,k,K,N,zipf", [
    (16384, 64, 8, 768, 512, True),      # 64 x 4 x 3 = 768 tiles, ragged / empty experts
    (16384, 8, 2, 2304, 1280, False),    # 8 x 10 x 9 = 720 tiles, several bands per expert
    (32768, 16, 2, 512, 1536, False),    # 16 x 12 x 2 = 384 tiles with the band over the other operand
])
def test_group_bwd_w_many_tiles_per_cta(T, E, k, K, N, zipf, gathered):
    from scattermoe_b200.kernels import ops
    if zipf:
        idx, g = _zipf_routing(T, E, k, seed=T + E + 2)
    else:
        _, idx, g = _routing(T, E, k, seed=T + E + K + 2)
    se, ss, off = oracle.flatten_sort_count(idx, E)
    DY = torch.randn(T * k, N, generator=g).bfloat16()
    if gathered:
        X = torch.randn(T, K, generator=g).bfloat16()
        Xg = oracle.group(X, ss, fan_out=k)
    else:
        Xg = X = torch.randn(T * k, K, generator=g).bfloat16()
    ops.FORCE_PATH = "tc"
    DW, Db = ops.group_bwd_W(_dev(DY), _dev(X), _dev(off), E, has_bias=True,
                             x_gather_idx=_dev(ss) if gathered else None, fan_out=k if gathered else 1)
    assert ops.last_path_was_tensor_core()
    wDW, wDb = oracle.group_bwd_W(DY.float(), Xg.float(), off, E, has_bias=True)
    counts = torch.bincount(idx.flatten(), minlength=E).clamp(min=1).float()
    scale = counts.sqrt().view(E, 1, 1)               # sums over the expert's rows of unit-variance products
    assert_close("DW", DW.float().cpu() / scale, wDW / scale, True)
    assert_close("Db", Db.float().cpu() / scale.view(E, 1), wDb / scale.view(E, 1), True)


@pytest.mark.parametrize("path", ["tc", "simt"])
@pytest.mark.parametrize("layout,act", [("plain", "gelu"), ("glu_second", "silu"), ("glu_first", "gelu"), ("gpt_oss", None)])
@pytest.mark.parametrize("T,E,k,K,F", [(513, 8, 3, 320, 200), (1000, 8, 2, 256, 384), (16384, 8, 4, 128, 512)])
def test_fused_epilogues_with_gates(T, E, k, K, F, layout, act, path):
    """Gates inside the fused epilogues: the up-projection kernel writes hidden * gate (the up-projection itself
    un-weighted); the gradient kernel takes the UN-weighted output gradient, scales the hidden gradient by the gate
    and returns the gate gradient <hidden, d_hidden> (the reference's `output_expanded @ grad_out`,
    parallel_experts.py:79, taken on the other side of the linear down-projection). The last shape makes every CTA
    walk several tiles."""
    from scattermoe_b200.kernels import ops
    dtype = torch.bfloat16
    n_up = F if layout == "plain" else 2 * F
    gates, idx, g = _routing(T, E, k, seed=T + K + F + 9, skew=True)
    gates = gates.to(dtype)
    se, ss, off = oracle.flatten_sort_count(idx, E)
    R = T * k
    lay, code = _act_codes(layout, act)
    X = torch.randn(T, K, generator=g).to(dtype)
    W1 = (torch.randn(E, n_up, K, generator=g) * 0.1).to(dtype).permute(0, 2, 1)
    row_g = gates.float().reshape(-1)[ss].unsqueeze(1)                  # gate of every expert-ordered row
    # forward
    ops.FORCE_PATH = None
    res = ops.scatter2scatter_act(_dev(X), _dev(W1), _dev(se), _dev(ss), k, lay, code, expert_offsets=_dev(off),
                                  row_gates=_dev(gates))
    assert res is not None
    up, hidden = res
    want_up = oracle.scatter2scatter(X.float(), W1.float(), se, ss, k, y_grouped=True)
    want_h = _act_reference(layout, act, want_up)
    assert_close("up", up, want_up, True)
    assert_close("hidden * gate", hidden, want_h * row_g, True, atol_scale=max(1.0, want_h.abs().max().item() / 4))
    # backward
    DY = torch.randn(R, K, generator=g).to(dtype)                        # un-weighted output gradient, expert order
    W2t = (torch.randn(E, K, F, generator=g) * 0.1).to(dtype)
    ops.FORCE_PATH = path if path == "simt" else None
    d_up, d_gates = ops.scatter2scatter_act_bwd(_dev(DY), _dev(W2t), up, _dev(off), lay, code, row_gates=_dev(gates),
                                                sorted_scattered_idxs=_dev(ss))
    if path == "tc":
        assert ops.last_path_was_tensor_core()
    d_hidden0 = oracle.scatter2scatter(DY.float(), W2t.float(), se, ss, 1, x_grouped=True, y_grouped=True)
    ref_in = up.float().cpu().requires_grad_()
    h_ref = _act_reference(layout, act, ref_in)
    (want_d_up,) = torch.autograd.grad(h_ref, ref_in, d_hidden0 * row_g)
    want_dg = torch.empty(R)
    want_dg[ss] = (h_ref.detach() * d_hidden0).sum(-1)
    assert_close("d_up", d_up, want_d_up, True, atol_scale=max(1.0, want_d_up.abs().max().item() / 4))
    assert d_gates.shape == (R,)
    scale = max(1.0, float(want_dg.pow(2).mean().sqrt()))              # a dot product of F bf16-rounded products
    assert_close("d_gates", d_gates.float().cpu() / scale, want_dg / scale, True)
