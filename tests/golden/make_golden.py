"""Generate the golden vectors under tests/golden/ by running the REFERENCE package.

Run where the reference project is checked out; pass its directory with --reference or $SCATTERMOE_REFERENCE:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --reference <path to the scattermoe checkout>

The reference's Triton kernels are executed on CPU tensors by the Triton interpreter, so the
stored outputs are outputs of the reference's own code path (scatter2scatter, group,
group_bwd_W, ParallelLinear forward/backward, MLP, GLUMLP and the two Hugging Face patches),
not of a restatement. Inputs come from seeded torch generators and are stored beside the
outputs, so the tests never need the reference at run time.

Cases flagged `bf16` hold inputs that are exactly representable in bfloat16 (generated, rounded to bf16,
widened back to float32) and outputs the reference computed from them in float32: the Triton interpreter
of this Triton release does not store bf16 tensors correctly, so the reference cannot be run in bf16 on a
CPU. An implementation under test runs those cases in bf16 and is compared with the bf16 tolerance
(rtol 2e-2 / atol 2e-2). Index tensors are stored as int64.
"""
import argparse
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))


def npy(t):
    if t is None:
        return None
    t = t.detach()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    return t.cpu().numpy()


def save(name, **arrays):
    arrays = {k: v for k, v in arrays.items() if v is not None}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
    print("wrote", name, {k: getattr(v, "shape", v) for k, v in arrays.items()})


def routing(gen, T, E, k, renorm=True, skew=False):
    logits = torch.randn(T, E, generator=gen)
    if skew:
        logits[:, : max(1, E // 4)] -= 20.0   # leaves some experts empty
    p = torch.softmax(logits, -1)
    w, idx = torch.topk(p, k)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("SCATTERMOE_REFERENCE"), required="SCATTERMOE_REFERENCE" not in os.environ)
    ap.add_argument("--only", choices=["single"], default=None,
                    help="regenerate one group of fixtures instead of all of them")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import scattermoe
    from scattermoe.kernels import ops
    from scattermoe.mlp import MLP, GLUMLP
    ops.ALLOW_TF32 = False

    # ---- single-token kernel (kernels/single.py:41): one or k input rows, both weight orientations --------
    from scattermoe.kernels.single import single2scatter
    for i, (E, k, K, N, x_rows, n_major) in enumerate([(4, 2, 128, 256, 1, True), (8, 4, 256, 128, 4, False),
                                                       (8, 3, 384, 256, 1, False)]):
        gen = torch.Generator().manual_seed(700 + i)
        X = torch.randn(x_rows, K, generator=gen)
        W = torch.randn(E, K, N, generator=gen) * 0.1 if n_major else (torch.randn(E, N, K, generator=gen) * 0.1).permute(0, 2, 1)
        idx = torch.randperm(E, generator=gen)[:k].view(1, k)
        Y = single2scatter(X, W, idx)
        save(f"single_{i}", X=npy(X), W=npy(W.contiguous()), expert_idxs=npy(idx), w_n_contiguous=np.bool_(n_major), Y=npy(Y))
    if args.only == "single":
        return

    # ---- routing bookkeeping -----------------------------------------------------------
    gen = torch.Generator().manual_seed(0)
    for i, (T, E, k, skew) in enumerate([(1, 8, 2, False), (256, 8, 2, False), (257, 32, 4, True),
                                          (4099, 64, 8, True), (1000, 128, 8, False), (3, 5, 5, False)]):
        _, idx = routing(gen, T, E, k, skew=skew)
        se, ss, off = scattermoe.flatten_sort_count(idx, num_experts=E)
        se2, ss2 = torch.sort(idx.flatten(), stable=True)
        save(f"sort_{i}", expert_idxs=npy(idx), E=np.int64(E), sorted_expert_idxs=npy(se),
             sorted_scattered_idxs=npy(ss), expert_offsets=npy(off),
             reference_was_stable=np.bool_(torch.equal(ss, ss2)))

    # ---- scatter2scatter, all four modes, both weight orientations, bias ----------------
    case = 0
    for dtype in (torch.float32, torch.bfloat16):
        for (T, E, k, K, N) in [(37, 4, 2, 72, 40), (130, 8, 3, 64, 136)]:
            for x_grouped in (False, True):
                for y_grouped in (False, True):
                    gen = torch.Generator().manual_seed(100 + case)
                    _, idx = routing(gen, T, E, k, skew=(case % 3 == 0))
                    se, ss, off = scattermoe.flatten_sort_count(idx, num_experts=E)
                    rows = T * k if x_grouped else T
                    kk = 1 if x_grouped else k
                    X = torch.randn(rows, K, generator=gen).to(dtype).float()
                    n_major = (case % 2 == 0)
                    if n_major:
                        W = (torch.randn(E, K, N, generator=gen) * 0.1).to(dtype).float()
                    else:
                        W = (torch.randn(E, N, K, generator=gen) * 0.1).to(dtype).float().permute(0, 2, 1)
                    b = (torch.randn(E, N, generator=gen) * 0.1).to(dtype).float() if case % 4 < 2 else None
                    Y = ops.scatter2scatter(X, W, se, ss, kk, b=b, x_grouped=x_grouped, y_grouped=y_grouped)
                    save(f"s2s_{case}", X=npy(X), W=npy(W.contiguous()), b=npy(b), expert_idxs=npy(idx),
                         E=np.int64(E), k=np.int64(kk), x_grouped=np.bool_(x_grouped), y_grouped=np.bool_(y_grouped),
                         w_n_contiguous=np.bool_(n_major), bf16=np.bool_(dtype == torch.bfloat16), Y=npy(Y),
                         sorted_expert_idxs=npy(se), sorted_scattered_idxs=npy(ss), expert_offsets=npy(off))
                    case += 1

    # ---- group ------------------------------------------------------------------------
    for i, (dtype, T, E, k, K, with_coeff) in enumerate([(torch.float32, 33, 4, 2, 50, True),
                                                         (torch.bfloat16, 65, 8, 4, 64, True),
                                                         (torch.float32, 17, 4, 3, 24, False)]):
        gen = torch.Generator().manual_seed(200 + i)
        w, idx = routing(gen, T, E, k)
        se, ss, off = scattermoe.flatten_sort_count(idx, num_experts=E)
        A = torch.randn(T, K, generator=gen).to(dtype).float()
        coeff = w.to(dtype).float().flatten() if with_coeff else None
        Y = ops.group(A, ss, coeff=coeff, fan_out=k)
        save(f"group_{i}", A=npy(A), coeff=npy(coeff), expert_idxs=npy(idx), E=np.int64(E), k=np.int64(k),
             bf16=np.bool_(dtype == torch.bfloat16), Y=npy(Y),
             sorted_expert_idxs=npy(se), sorted_scattered_idxs=npy(ss), expert_offsets=npy(off))

    # ---- group_bwd_W (with an empty expert and bias) ------------------------------------
    for i, (dtype, T, E, k, K, N, has_bias) in enumerate([(torch.float32, 61, 8, 2, 40, 72, True),
                                                          (torch.bfloat16, 200, 4, 2, 64, 128, False),
                                                          (torch.float32, 2, 8, 2, 136, 24, True)]):
        gen = torch.Generator().manual_seed(300 + i)
        _, idx = routing(gen, T, E, k, skew=True)
        se, ss, off = scattermoe.flatten_sort_count(idx, num_experts=E)
        X = torch.randn(T * k, K, generator=gen).to(dtype).float()
        DY = torch.randn(T * k, N, generator=gen).to(dtype).float()
        DW, Db = ops.group_bwd_W(DY, X, off, E, has_bias=has_bias)
        save(f"gbw_{i}", X=npy(X), DY=npy(DY), expert_idxs=npy(idx), E=np.int64(E),
             bf16=np.bool_(dtype == torch.bfloat16), DW=npy(DW.contiguous()), Db=npy(Db),
             sorted_expert_idxs=npy(se), sorted_scattered_idxs=npy(ss), expert_offsets=npy(off))

    # ---- MLP / GLUMLP forward + backward ------------------------------------------------
    def run_module(name, mod, T, E, k, d, dtype, seed, renorm):
        gen = torch.Generator().manual_seed(seed)
        w, idx = routing(gen, T, E, k, renorm=renorm)
        w = w.to(dtype).float().requires_grad_()
        X = torch.randn(T, d, generator=gen).to(dtype).float().requires_grad_()
        DY = torch.randn(T, d, generator=gen).to(dtype).float()
        with torch.no_grad():
            for p in mod.parameters():
                p.copy_((torch.randn(p.shape, generator=gen) * (0.05 if p.dim() == 3 else 0.02)).to(dtype).float())
        Y = mod(X, w, idx)
        params = dict(mod.named_parameters())
        leaves = [X, w] + list(params.values())
        grads = torch.autograd.grad(Y, leaves, DY)
        out = dict(X=npy(X), expert_p=npy(w), expert_idxs=npy(idx), DY=npy(DY), Y=npy(Y),
                   dX=npy(grads[0]), d_expert_p=npy(grads[1]), E=np.int64(E), k=np.int64(k),
                   bf16=np.bool_(dtype == torch.bfloat16))
        for (n, p), g in zip(params.items(), grads[2:]):
            out["param." + n] = npy(p)
            out["grad." + n] = npy(g)
        save(name, **out)

    run_module("mlp_gelu_fp32", MLP(64, 96, 8, 2, activation=nn.GELU()), 96, 8, 2, 64, torch.float32, 400, False)
    run_module("mlp_gelu_fp32_bias", MLP(100, 133, 8, 3, bias=True, activation=nn.GELU()), 50, 8, 3, 100, torch.float32, 401, False)
    run_module("mlp_gelu_fp32_T1", MLP(64, 128, 8, 4, bias=True, activation=nn.GELU()), 1, 8, 4, 64, torch.float32, 402, True)
    run_module("glumlp_silu_fp32", GLUMLP(64, 48, 8, 2), 80, 8, 2, 64, torch.float32, 403, True)
    run_module("glumlp_silu_bf16", GLUMLP(128, 64, 4, 2), 160, 4, 2, 128, torch.bfloat16, 404, True)
    run_module("mlp_gelu_bf16", MLP(128, 256, 8, 2, activation=nn.GELU()), 128, 8, 2, 128, torch.bfloat16, 405, True)

    # ---- Hugging Face patches ------------------------------------------------------------
    # The patched forwards are installed on the HF classes when the reference is imported.
    try:
        from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts
        from transformers.models.gpt_oss.configuration_gpt_oss import GptOssConfig
        cfg = GptOssConfig(hidden_size=64, intermediate_size=48, num_local_experts=8, num_experts_per_tok=4,
                           num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=32)
        gen = torch.Generator().manual_seed(500)
        ex = GptOssExperts(cfg)
        with torch.no_grad():
            for p in ex.parameters():
                p.copy_(torch.randn(p.shape, generator=gen) * 0.05)
        T = 40
        hs = torch.randn(2, T // 2, 64, generator=gen).requires_grad_()
        logits = torch.randn(T, 8, generator=gen)
        top, ridx = torch.topk(logits, 4, dim=-1)
        scores = torch.softmax(top, dim=-1)
        # the reference patch gathers from a (T, E) score matrix (replace_moe.py:26)
        full = torch.zeros(T, 8).scatter_(1, ridx, scores).requires_grad_()
        out = GptOssExperts.forward(ex, hs, router_indices=ridx, routing_weights=full)
        DY = torch.randn(out.shape, generator=gen)
        params = dict(ex.named_parameters())
        grads = torch.autograd.grad(out, [hs, full] + list(params.values()), DY)
        d = dict(hidden_states=npy(hs), router_indices=npy(ridx), routing_weights_full=npy(full),
                 routing_weights_topk=npy(scores), DY=npy(DY), Y=npy(out), d_hidden_states=npy(grads[0]),
                 d_routing_weights_topk=npy(torch.gather(grads[1], 1, ridx)))
        for (n, p), g in zip(params.items(), grads[2:]):
            d["param." + n] = npy(p)
            d["grad." + n] = npy(g)
        save("hf_gpt_oss_experts", **d)
    except Exception as e:  # pragma: no cover
        print("gpt_oss golden skipped:", repr(e))

    try:
        from transformers.models.granitemoehybrid.modeling_granitemoehybrid import GraniteMoeHybridMoE
        from transformers.models.granitemoehybrid.configuration_granitemoehybrid import GraniteMoeHybridConfig
        cfg = GraniteMoeHybridConfig(hidden_size=64, intermediate_size=48, num_local_experts=8,
                                     num_experts_per_tok=2, num_hidden_layers=1, num_attention_heads=2,
                                     num_key_value_heads=1, shared_intermediate_size=32)
        gen = torch.Generator().manual_seed(501)
        moe = GraniteMoeHybridMoE(cfg)
        with torch.no_grad():
            for p in moe.parameters():
                p.copy_(torch.randn(p.shape, generator=gen) * 0.05)
        x = torch.randn(2, 24, 64, generator=gen).requires_grad_()
        res = GraniteMoeHybridMoE.forward(moe, x)
        out, router_logits = res if isinstance(res, tuple) else (res, None)
        DY = torch.randn(out.shape, generator=gen)
        params = dict(moe.named_parameters())
        grads = torch.autograd.grad(out, [x] + list(params.values()), DY)
        d = dict(layer_input=npy(x), DY=npy(DY), Y=npy(out), router_logits=npy(router_logits), dX=npy(grads[0]))
        for (n, p), g in zip(params.items(), grads[1:]):
            d["param." + n] = npy(p)
            d["grad." + n] = npy(g)
        save("hf_granitemoehybrid_moe", **d)
    except Exception as e:  # pragma: no cover
        print("granite golden skipped:", repr(e))


if __name__ == "__main__":
    main()
