"""Module-level parity on the GPU: MLP / GLUMLP / ParallelExperts / the Hugging Face patches against the
reference's golden outputs and the dense per-expert oracle, forward and every gradient."""
import os
import sys

import pytest
import torch
from torch import nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import scattermoe_oracle as oracle  # noqa: E402
from util import assert_close, load_golden  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    import scattermoe_b200 as sm
    from scattermoe_b200.kernels import ops
    ops.FORCE_PATH = None
    ops.ALLOW_TF32 = True
    yield
    ops.FORCE_PATH = None
    sm.check_device_status()


def _load_module(g, cls, **kw):
    import scattermoe_b200 as sm
    w1 = g["param.experts.weight"]
    w2 = g["param.output_experts.weight"]
    E, d = w1.shape[0], w1.shape[2]
    hidden = w2.shape[2]
    bias = "param.experts.bias" in g
    m = getattr(sm.mlp, cls)(d, hidden, E, g["k"], bias=bias, **kw)
    sd = {k[len("param."):]: v for k, v in g.items() if k.startswith("param.")}
    m.load_state_dict(sd)
    dt = torch.bfloat16 if g["bf16"] else torch.float32
    return m.cuda().to(dt), dt


@pytest.mark.parametrize("name,cls,kw", [
    ("mlp_gelu_fp32", "MLP", dict(activation=nn.GELU())),
    ("mlp_gelu_fp32_bias", "MLP", dict(activation=nn.GELU())),
    ("mlp_gelu_fp32_T1", "MLP", dict(activation=nn.GELU())),
    ("glumlp_silu_fp32", "GLUMLP", {}),
    ("glumlp_silu_bf16", "GLUMLP", {}),
    ("mlp_gelu_bf16", "MLP", dict(activation=nn.GELU())),
])
def test_module_golden(name, cls, kw):
    g = load_golden(name)
    m, dt = _load_module(g, cls, **kw)
    X = g["X"].to(dt).cuda().requires_grad_()
    p = g["expert_p"].to(dt).cuda().requires_grad_()
    Y = m(X, p, g["expert_idxs"].cuda())
    params = dict(m.named_parameters())
    grads = torch.autograd.grad(Y, [X, p] + list(params.values()), g["DY"].to(dt).cuda())
    bf16 = g["bf16"]

    def scale(ref):
        # bf16 cases: the stored outputs are fp32 results, the run under test rounds every intermediate to
        # bf16 as the reference's bf16 run does; gradients are sums of many such terms with magnitudes of
        # several units, so the absolute tolerance is applied after bringing them to unit scale.
        return max(1.0, ref.abs().max().item() / 4) if bf16 else 1.0

    assert_close(name + ".Y", Y, g["Y"], bf16)
    assert_close(name + ".dX", grads[0], g["dX"], bf16, atol_scale=scale(g["dX"]))
    assert_close(name + ".dg", grads[1], g["d_expert_p"], bf16, atol_scale=scale(g["d_expert_p"]))
    for (n, _), gr in zip(params.items(), grads[2:]):
        assert_close(name + ".grad." + n, gr, g["grad." + n], bf16, atol_scale=scale(g["grad." + n]))


# The reference's own test grid (tests/test_mlp.py:36-44): fp32, E=8, GELU, TF32 off, max abs diff < 1e-4
# on Y, dX, d(gates), dW1, dW2 (and both bias grads), against the dense loop.
GRID = [(xd, (4 * xd) // k, k) for xd in [128, 256, 512, 600, 100] for k in [2, 3, 4]]


@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("length", [1, 256, 512])
@pytest.mark.parametrize("x_dim,h_dim,k", GRID)
def test_reference_test_grid(length, x_dim, h_dim, k, bias):
    import scattermoe_b200 as sm
    sm.kernels.ops.ALLOW_TF32 = False
    E = 8
    g = torch.Generator().manual_seed(length * 7 + x_dim + k + int(bias))
    logits = torch.randn(length, E, generator=g)
    weights = torch.softmax(logits, dim=-1)
    k_weights, k_idxs = torch.topk(weights, k)      # no renormalisation, as in the reference test
    X = torch.randn(length, x_dim, generator=g)
    DY = torch.randn(length, x_dim, generator=g)
    torch.manual_seed(0)
    m = sm.mlp.MLP(x_dim, h_dim, E, k, bias=bias, activation=nn.GELU())
    if bias:
        nn.init.normal_(m.experts.bias, std=0.02)
        nn.init.normal_(m.output_experts.bias, std=0.02)
    w1, w2 = m.experts.weight.detach().clone(), m.output_experts.weight.detach().clone()
    b1 = m.experts.bias.detach().clone() if bias else None
    b2 = m.output_experts.bias.detach().clone() if bias else None
    m = m.cuda()
    Xc = X.cuda().requires_grad_()
    pc = k_weights.cuda().requires_grad_()
    Y = m(Xc, pc, k_idxs.cuda())
    params = dict(m.named_parameters())
    grads = torch.autograd.grad(Y, [Xc, pc] + list(params.values()), DY.cuda())
    want = oracle.moe_mlp_forward_backward(X, k_weights, k_idxs, w1.permute(0, 2, 1), w2.permute(0, 2, 1), b1, b2,
                                           oracle.act_gelu, DY)
    assert_close("Y", Y, want["y"], False)
    assert_close("dX", grads[0], want["d_x"], False)
    assert_close("dg", grads[1], want["d_expert_p"], False)
    got = dict(zip(params.keys(), grads[2:]))
    assert_close("dW1", got["experts.weight"], want["d_w1"].permute(0, 2, 1), False)
    assert_close("dW2", got["output_experts.weight"], want["d_w2"].permute(0, 2, 1), False)
    if bias:
        assert_close("db1", got["experts.bias"], want["d_b1"], False)
        assert_close("db2", got["output_experts.bias"], want["d_b2"], False)


@pytest.mark.parametrize("group_copy,gather_rows", [(True, False), (False, False), (False, True)])
def test_input_feeding_variants_agree(group_copy, gather_rows):
    """The three ways the tensor-core kernels can be fed (expert-order copy + TMA, in-kernel cp.async row gather
    of the un-grouped input, cp.async gather of grouped inputs too) give the same layer outputs and gradients."""
    import scattermoe_b200 as sm
    from scattermoe_b200 import parallel_experts as pe
    from scattermoe_b200.kernels import ops
    torch.manual_seed(3)
    T, d, F, E, k = 777, 256, 192, 8, 2
    m = sm.mlp.GLUMLP(d, F, E, k).cuda().bfloat16()
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)
    p, idx = torch.topk(torch.softmax(torch.randn(T, E, device="cuda"), -1), k)
    dy = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)

    def run():
        xx, pp = x.clone().requires_grad_(), p.bfloat16().requires_grad_()
        y = m(xx, pp, idx)
        return [y] + list(torch.autograd.grad(y, [xx, pp, m.experts.weight, m.output_experts.weight], dy))
    base = run()
    old = pe.GROUP_INPUT_COPY
    try:
        pe.GROUP_INPUT_COPY, ops.GATHER_ROWS = group_copy, gather_rows
        got = run()
    finally:
        pe.GROUP_INPUT_COPY, ops.GATHER_ROWS = old, False
    for a, b in zip(got, base):
        torch.testing.assert_close(a.float(), b.float(), rtol=1e-2, atol=1e-2 * max(1.0, b.float().abs().max().item()))


def test_leading_shape_is_restored_and_grouped_flags():
    import scattermoe_b200 as sm
    torch.manual_seed(1)
    m = sm.mlp.GLUMLP(64, 32, 4, 2).cuda().bfloat16()
    x = torch.randn(2, 5, 64, device="cuda", dtype=torch.bfloat16)
    p = torch.softmax(torch.randn(10, 4, device="cuda"), -1)
    w, idx = torch.topk(p, 2)
    y = m(x, w.bfloat16(), idx)
    assert y.shape == (2, 5, 64)


def test_hf_gpt_oss_patch_golden():
    import scattermoe_b200  # noqa: F401  (installs the patch)
    from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts
    from transformers.models.gpt_oss.configuration_gpt_oss import GptOssConfig
    g = load_golden("hf_gpt_oss_experts")
    cfg = GptOssConfig(hidden_size=64, intermediate_size=48, num_local_experts=8, num_experts_per_tok=4,
                       num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=32)
    ex = GptOssExperts(cfg)
    ex.load_state_dict({k[len("param."):]: v for k, v in g.items() if k.startswith("param.")})
    ex = ex.cuda()
    for rw_key in ("routing_weights_topk", "routing_weights_full"):     # (T,k) of new routers, (T,E) of old ones
        hs = g["hidden_states"].cuda().requires_grad_()
        rw = g[rw_key].cuda().requires_grad_()
        out = ex(hs, router_indices=g["router_indices"].cuda(), routing_weights=rw)
        params = dict(ex.named_parameters())
        grads = torch.autograd.grad(out, [hs, rw] + list(params.values()), g["DY"].cuda())
        assert_close("Y", out, g["Y"], False)
        assert_close("dX", grads[0], g["d_hidden_states"], False)
        d_rw = grads[1] if rw_key.endswith("topk") else torch.gather(grads[1], 1, g["router_indices"].cuda())
        assert_close("dg", d_rw, g["d_routing_weights_topk"], False)
        for (n, _), gr in zip(params.items(), grads[2:]):
            assert_close("grad." + n, gr, g["grad." + n], False)


def test_hf_granite_patch_golden():
    import scattermoe_b200 as sm
    from transformers.models.granitemoehybrid.modeling_granitemoehybrid import GraniteMoeHybridMoE
    from transformers.models.granitemoehybrid.configuration_granitemoehybrid import GraniteMoeHybridConfig
    g = load_golden("hf_granitemoehybrid_moe")
    cfg = GraniteMoeHybridConfig(hidden_size=64, intermediate_size=48, num_local_experts=8, num_experts_per_tok=2,
                                 num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                                 shared_intermediate_size=32)
    moe = GraniteMoeHybridMoE(cfg)
    moe.load_state_dict({k[len("param."):]: v for k, v in g.items() if k.startswith("param.")})
    moe = moe.cuda()
    x = g["layer_input"].cuda().requires_grad_()
    res = moe(x)
    if sm.utils.replace_moe.GRANITE_RETURNS_ROUTER_LOGITS:
        out, logits = res
        assert_close("router_logits", logits, g["router_logits"], False)
    else:
        out = res
        assert torch.is_tensor(out)
    params = dict(moe.named_parameters())
    grads = torch.autograd.grad(out, [x] + list(params.values()), g["DY"].cuda())
    assert_close("Y", out, g["Y"], False)
    assert_close("dX", grads[0], g["dX"], False)
    for (n, _), gr in zip(params.items(), grads[1:]):
        assert_close("grad." + n, gr, g["grad." + n], False)


BF16_LAYERS = [
    # name, T, d, F, E, k, kind, bias
    ("glu", 1024, 512, 384, 8, 2, "glu_silu", False),
    ("gpt_oss", 512, 320, 320, 16, 4, "gpt_oss", True),
    ("zipf", 2048, 256, 128, 32, 8, "glu_silu", False),
]


@pytest.mark.parametrize("name,T,d,F,E,k,kind,bias", BF16_LAYERS)
def test_bf16_layers_against_fp32_dense_loop(name, T, d, F, E, k, kind, bias):
    """Scaled-down copies of the benchmark layers in bf16 on the tensor-core path against the fp32 dense
    loop on the same (bf16-rounded) inputs; rtol 2e-2 / atol 2e-2 after normalising gradients to unit scale."""
    import scattermoe_b200 as sm
    from scattermoe_b200.utils.replace_moe import gpt_oss_glu
    cfg = "granite_zipf" if name == "zipf" else ("gpt_oss_20b" if kind == "gpt_oss" else "mixtral_8x7b")
    p, idx = oracle.make_routing(cfg, T, E, k, seed=1)
    g = torch.Generator().manual_seed(2)
    bf = torch.bfloat16
    n1 = 2 * F
    x = torch.randn(T, d, generator=g).to(bf)
    w1 = (torch.randn(E, d, n1, generator=g) * 0.05).to(bf)
    w2 = (torch.randn(E, F, d, generator=g) * 0.05).to(bf)
    b1 = (torch.randn(E, n1, generator=g) * 0.02).to(bf) if bias else None
    b2 = (torch.randn(E, d, generator=g) * 0.02).to(bf) if bias else None
    go = torch.randn(T, d, generator=g).to(bf)
    p = p.to(bf)
    act = oracle.act_gpt_oss if kind == "gpt_oss" else oracle.act_glu_second_half
    want = oracle.moe_mlp_forward_backward(x, p, idx, w1, w2, b1, b2, act, go, compute_dtype=torch.float32)

    leaves = [t.cuda().requires_grad_() for t in (x, p, w1, w2)]
    xb, pb, w1b, w2b = leaves
    bl = [t.cuda().requires_grad_() for t in (b1, b2)] if bias else []
    routing = sm.flatten_sort_count(idx.cuda(), E)
    up = sm.parallel_linear(xb, w1b, k, *routing, expert_biases=bl[0] if bias else None, grouped_out=True)
    if kind == "gpt_oss":
        h = gpt_oss_glu(up, 1.702, 7.0)
    else:
        lin, gate = up.chunk(2, dim=-1)
        h = torch.nn.functional.silu(gate) * lin
    y = sm.parallel_linear(h, w2b, 1, *routing, expert_biases=bl[1] if bias else None, grouped_in=True, gates=pb)
    grads = torch.autograd.grad(y, leaves + bl, go.cuda())
    assert sm.kernels.ops.last_path_was_tensor_core()

    def cmp(nm, got, ref):
        s = max(ref.abs().max().item(), 1e-6) if nm != "y" else 1.0
        s = max(s / 4, 1.0) if nm != "y" else 1.0
        assert_close(nm, got.float().cpu() / s, ref / s, True)
    cmp("y", y, want["y"])
    cmp("dx", grads[0], want["d_x"])
    cmp("dp", grads[1], want["d_expert_p"])
    cmp("dw1", grads[2], want["d_w1"])
    cmp("dw2", grads[3], want["d_w2"])
    if bias:
        cmp("db1", grads[4], want["d_b1"])
        cmp("db2", grads[5], want["d_b2"])


def test_module_runs_under_torch_compile():
    """The reference advertises its layer as usable inside torch.compile (README changelog 0.2.0). The whole layer
    must trace as one graph (fullgraph=True raises on any graph break), forward and backward, with results
    bit-equal to the eager ones."""
    import scattermoe_b200 as sm
    torch.manual_seed(0)
    m = sm.mlp.GLUMLP(256, 128, 8, 2).cuda().bfloat16()
    x = torch.randn(300, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    p, idx = torch.topk(torch.softmax(torch.randn(300, 8, device="cuda"), -1), 2)
    p = p.bfloat16().requires_grad_()
    leaves = [x, p, m.experts.weight, m.output_experts.weight]
    y0 = m(x, p, idx)
    g0 = torch.autograd.grad(y0, leaves, torch.ones_like(y0))
    compiled = torch.compile(m, fullgraph=True)
    y1 = compiled(x, p, idx)
    g1 = torch.autograd.grad(y1, leaves, torch.ones_like(y1))
    assert torch.equal(y1, y0)
    for a, b in zip(g1, g0):
        assert torch.equal(a, b)


@pytest.mark.parametrize("family", ["qwen3_moe", "mixtral"])
def test_hf_fused_expert_blocks(family):
    """Qwen3-MoE / Mixtral expert blocks of current transformers releases (fused 3-D expert tensors) routed through
    the grouped-GEMM path, against Hugging Face's own per-expert loop in fp32 on the CPU, forward and gradients."""
    import copy
    import scattermoe_b200 as sm
    if family == "qwen3_moe":
        from transformers.models.qwen3_moe.modeling_qwen3_moe import Qwen3MoeExperts as Experts
        from transformers.models.qwen3_moe.configuration_qwen3_moe import Qwen3MoeConfig
        cfg = Qwen3MoeConfig(hidden_size=64, moe_intermediate_size=48, num_experts=8, num_experts_per_tok=2,
                             num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, intermediate_size=64)
    else:
        from transformers.models.mixtral.modeling_mixtral import MixtralExperts as Experts
        from transformers.models.mixtral.configuration_mixtral import MixtralConfig
        cfg = MixtralConfig(hidden_size=64, intermediate_size=48, num_local_experts=8, num_experts_per_tok=2,
                            num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1)
    assert Experts.__name__ in sm.utils.replace_moe.PATCHED
    g = torch.Generator().manual_seed(9)
    ex = Experts(cfg)
    with torch.no_grad():
        for p in ex.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    T = 50
    x = torch.randn(T, 64, generator=g)
    w, idx = torch.topk(torch.softmax(torch.randn(T, 8, generator=g), -1), 2)
    dy = torch.randn(T, 64, generator=g)

    def run(mod, dev):
        xx, ww = x.to(dev).requires_grad_(), w.to(dev).requires_grad_()
        y = mod(xx, idx.to(dev), ww)
        grads = torch.autograd.grad(y, [xx, ww] + list(mod.parameters()), dy.to(dev))
        return [y] + list(grads)
    want = run(ex, "cpu")                      # CPU tensors take Hugging Face's own forward
    got = run(copy.deepcopy(ex).cuda(), "cuda")
    for name, a, b in zip(("y", "dx", "dw", "d_gate_up", "d_down"), got, want):
        assert_close(name, a, b, False)


def _glu_reference(x, p, idx, w1, w2, dy):
    return oracle.moe_mlp_forward_backward(x, p, idx, w1.permute(0, 2, 1), w2.permute(0, 2, 1), None, None,
                                           oracle.act_glu_second_half, dy, compute_dtype=torch.float32)


@pytest.mark.parametrize("case", ["one_expert_takes_all", "fp16", "strided_input", "more_experts_than_the_tc_table"])
def test_edge_cases_against_the_dense_loop(case):
    """Ragged extremes and input layouts the reference's masks handle implicitly: every token to one expert (all
    other segments empty), fp16, an input that is a strided view, and an expert count beyond the tensor-core
    kernel's segment table (the CUDA-core kernels take over)."""
    import scattermoe_b200 as sm
    dtype = torch.float16 if case == "fp16" else torch.bfloat16
    T, d, F, k = 200, 128, 72, 2
    E = 1100 if case == "more_experts_than_the_tc_table" else 8
    g = torch.Generator().manual_seed(len(case))
    x = torch.randn(T, d, generator=g).to(dtype)
    if case == "one_expert_takes_all":
        idx = torch.full((T, k), 5, dtype=torch.int64)
        idx[:, 1] = 2
        idx[:, 0] = 5
        idx[:, 1] = 5        # both slots of every token go to expert 5
    else:
        idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    p = torch.rand(T, k, generator=g).to(dtype)
    w1 = (torch.randn(E, 2 * F, d, generator=g) * 0.05).to(dtype)
    w2 = (torch.randn(E, d, F, generator=g) * 0.05).to(dtype)
    dy = torch.randn(T, d, generator=g).to(dtype)
    want = _glu_reference(x, p, idx, w1, w2, dy)
    m = sm.mlp.GLUMLP(d, F, E, k).cuda().to(dtype)
    with torch.no_grad():
        m.experts.weight.copy_(w1)
        m.output_experts.weight.copy_(w2)
    if case == "strided_input":
        wide = torch.zeros(T, 2 * d, dtype=dtype, device="cuda")
        wide[:, ::2] = x.cuda()
        xd = wide[:, ::2].requires_grad_()          # inner stride 2
    else:
        xd = x.cuda().requires_grad_()
    pd = p.cuda().requires_grad_()
    y = m(xd, pd, idx.cuda())
    grads = torch.autograd.grad(y, [xd, pd, m.experts.weight, m.output_experts.weight], dy.cuda())

    def cmp(name, got, ref):
        s = max(1.0, ref.abs().max().item() / 4)
        assert_close(name, got.float().cpu() / s, ref / s, True)
    cmp("y", y, want["y"]); cmp("dx", grads[0], want["d_x"]); cmp("dp", grads[1], want["d_expert_p"])
    cmp("dw1", grads[2], want["d_w1"].permute(0, 2, 1)); cmp("dw2", grads[3], want["d_w2"].permute(0, 2, 1))
    if case == "one_expert_takes_all":
        untouched = [e for e in range(E) if e != 5]
        assert bool((grads[2][untouched] == 0).all()) and bool((grads[3][untouched] == 0).all())


def test_no_tokens_at_all():
    """T = 0: outputs are empty, weight gradients exact zeros, nothing is launched out of bounds."""
    import scattermoe_b200 as sm
    m = sm.mlp.GLUMLP(64, 48, 4, 2).cuda().bfloat16()
    x = torch.zeros(0, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    p = torch.zeros(0, 2, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    idx = torch.zeros(0, 2, device="cuda", dtype=torch.int64)
    y = m(x, p, idx)
    assert y.shape == (0, 64)
    gx, gw = torch.autograd.grad(y, [x, m.experts.weight], torch.zeros_like(y))
    assert gx.shape == (0, 64) and bool((gw == 0).all())


def test_layer_replays_from_a_cuda_graph():
    """A layer step is a fixed launch sequence (grids from host-known bounds, routing read on the device, no host
    synchronisation), so plain stream capture works: forward + backward captured once, replayed with different
    tokens AND different routing, equal to eager."""
    import scattermoe_b200 as sm
    torch.manual_seed(4)
    T, d, F, E, k = 256, 256, 192, 8, 2
    m = sm.mlp.GLUMLP(d, F, E, k).cuda().bfloat16()

    def inputs(seed):
        g = torch.Generator(device="cuda").manual_seed(seed)
        x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, generator=g).requires_grad_()
        p, idx = torch.topk(torch.softmax(torch.randn(T, E, device="cuda", generator=g), -1), k)
        return x, p.bfloat16().requires_grad_(), idx, torch.randn(T, d, device="cuda", dtype=torch.bfloat16, generator=g)
    x0, p0, i0, _ = inputs(0)
    graphed = torch.cuda.make_graphed_callables(m, (x0, p0, i0), num_warmup_iters=3, allow_unused_input=True)
    for seed in (1, 2):
        x, p, idx, dy = inputs(seed)
        y = graphed(x, p, idx)
        gx, gp = torch.autograd.grad(y, [x, p], dy)
        xe, pe = x.detach().clone().requires_grad_(), p.detach().clone().requires_grad_()
        ye = m(xe, pe, idx)
        gxe, gpe = torch.autograd.grad(ye, [xe, pe], dy)
        assert torch.equal(y, ye) and torch.equal(gx, gxe) and torch.equal(gp, gpe)
    sm.check_device_status()


@pytest.mark.parametrize("names_kind,renorm", [("qwen", True), ("qwen", False), ("mixtral", True)])
def test_consolidated_module_list_block(names_kind, renorm):
    """A sparse-MoE block whose experts are an nn.ModuleList (the layout the reference's abandoned Qwen3 patch was
    written for, replace_moe.py:97-208): after consolidation the block's forward and every gradient equal the
    per-expert loop over the original modules."""
    import scattermoe_b200 as sm
    from scattermoe_b200.utils import consolidate as C
    names = C.QWEN_NAMES if names_kind == "qwen" else C.MIXTRAL_NAMES
    torch.manual_seed(7)
    H, I, E, k, T = 256, 192, 8, 2, 300
    g_, u_, d_ = names

    class Expert(nn.Module):
        def __init__(self):
            super().__init__()
            setattr(self, g_, nn.Linear(H, I, bias=False))
            setattr(self, u_, nn.Linear(H, I, bias=False))
            setattr(self, d_, nn.Linear(I, H, bias=False))
            self.act_fn = nn.SiLU()

        def forward(self, x):
            return getattr(self, d_)(self.act_fn(getattr(self, g_)(x)) * getattr(self, u_)(x))

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate = nn.Linear(H, E, bias=False)
            self.experts = nn.ModuleList([Expert() for _ in range(E)])
            self.top_k, self.norm_topk_prob = k, renorm

    ref = Block().cuda().float()
    x = torch.randn(2, T // 2, H, device="cuda")
    dy = torch.randn_like(x)

    def loop_forward(block, inp):          # what Hugging Face's ModuleList blocks do: one expert at a time
        tokens = inp.reshape(-1, H)
        logits = block.gate(tokens)
        p = torch.softmax(logits, dim=-1, dtype=torch.float)
        w, ids = torch.topk(p, k, dim=-1)
        if renorm:
            w = w / w.sum(-1, keepdim=True)
        out = torch.zeros_like(tokens)
        for e in range(E):
            tok, slot = (ids == e).nonzero(as_tuple=True)
            if tok.numel():
                out = out.index_add(0, tok, block.experts[e](tokens[tok]) * w[tok, slot].unsqueeze(1))
        return out.view(inp.shape), logits

    xr = x.clone().requires_grad_()
    want_y, want_logits = loop_forward(ref, xr)
    want_params = dict(ref.named_parameters())
    want_grads = torch.autograd.grad(want_y, [xr] + list(want_params.values()), dy)
    want_sd = {n: t.detach().clone() for n, t in ref.state_dict().items()}

    fused = Block().cuda().float()
    fused.load_state_dict(want_sd)
    C.consolidate_moe_block(fused, names=names)
    xf = x.clone().requires_grad_()
    y, logits = C.moe_block_forward(fused, xf)
    torch.testing.assert_close(logits, want_logits)
    assert (y - want_y).abs().max().item() < 1e-4
    got = torch.autograd.grad(y, [xf, fused.gate.weight, fused.experts.gate_up_proj, fused.experts.down_proj], dy)
    assert (got[0] - want_grads[0]).abs().max().item() < 1e-4
    names_list = list(want_params)
    by_name = dict(zip(names_list, want_grads[1:]))
    assert (got[1] - by_name["gate.weight"]).abs().max().item() < 1e-4
    for e in range(E):
        assert (got[2][e, :I] - by_name["experts.%d.%s.weight" % (e, g_)]).abs().max().item() < 1e-4
        assert (got[2][e, I:] - by_name["experts.%d.%s.weight" % (e, u_)]).abs().max().item() < 1e-4
        assert (got[3][e] - by_name["experts.%d.%s.weight" % (e, d_)]).abs().max().item() < 1e-4
    # checkpoint of the consolidated block == checkpoint of the original
    sd = fused.state_dict()
    assert sorted(sd) == sorted(want_sd) and all(torch.equal(sd[n], want_sd[n]) for n in sd)
    sm.check_device_status()


def test_forward_without_gradients_equals_the_training_forward():
    """Under torch.no_grad the fused up-projection kernel does not write the up-projection (nothing needs it); the
    layer's output must be the same bits."""
    import scattermoe_b200 as sm
    torch.manual_seed(2)
    T, d, F, E, k = 1000, 256, 320, 8, 2
    m = sm.mlp.GLUMLP(d, F, E, k).cuda().bfloat16()
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)
    p, idx = torch.topk(torch.softmax(torch.randn(T, E, device="cuda"), -1), k)
    p = p.bfloat16()
    y_train = m(x.clone().requires_grad_(), p.clone().requires_grad_(), idx)
    with torch.no_grad():
        y_inf = m(x, p, idx)
    assert not y_inf.requires_grad and torch.equal(y_inf, y_train.detach())
    sm.check_device_status()
