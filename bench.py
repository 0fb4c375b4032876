"""Benchmark of the MoE-layer hot path: forward + backward tokens/s of one expert-MLP layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl ours|reference]

One "step" = routing bookkeeping (flatten_sort_count) + forward + backward (gradients w.r.t. the input, the
gates and both expert weight tensors) of the layer on one batch of seeded synthetic tokens. Prints ONE JSON
line. `value` is device-timed with the inputs resident in HBM; `e2e` repeats the measurement with every step's
inputs copied from pinned host memory and its results copied back inside the timed region; `forward` is the
forward pass alone. `parity` compares, outside the timed regions, the outputs and gradients of one full-size step
with the reference's own Triton kernels on the same GPU, weights and inputs, and a sample of token rows with an
fp32 dense per-expert loop. `other_configs` (N = 1) carries short measurements of the remaining single-GPU
workloads; `ep_config5` the expert-parallel workload at this N.

N > 1 (launched by torch.distributed.run, one rank per GPU): expert parallel, strong scaling. The layer's experts
are partitioned across the ranks, the workload's tokens are split evenly, and every step exchanges rows over
NVLink peer memory (scattermoe_b200.expert_parallel). Time is the max over ranks, `value` the global tokens per
second. (The gpt-oss workload, whose block has biases and its own activation, is not expert-parallel here: its
ranks run replicas on their own token shards, weak scaling.)

`--impl reference` times the reference's CPU path for the same layer (the dense per-expert PyTorch loop the
reference's own test uses as ground truth) on the host cores, every step on a bounded sample of the tokens.
"""
from __future__ import annotations

import argparse
import gc
import importlib
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = {
    # name: T, d_model, d_ffn, E, top_k, kind, bias
    "mixtral_8x7b": dict(T=16384, d=4096, F=14336, E=8, k=2, kind="glu_silu", bias=False),
    "gpt_oss_20b": dict(T=8192, d=2880, F=2880, E=32, k=4, kind="gpt_oss", bias=True),
    "granite_zipf": dict(T=32768, d=1536, F=512, E=64, k=8, kind="glu_silu", bias=False),
    "qwen3_moe_ep": dict(T=65536, d=2048, F=768, E=128, k=8, kind="glu_silu", bias=False),
    "tiny": dict(T=256, d=128, F=256, E=8, k=2, kind="glu_silu", bias=False),
}
CPU_SAMPLE_TOKENS = {"mixtral_8x7b": 2048, "gpt_oss_20b": 2048, "granite_zipf": 8192, "qwen3_moe_ep": 8192, "tiny": 256}
CPU_ARM_BUDGET_S = 240.0      # the whole `--impl reference` run (warm-up + steps) is sized to end within this
METRIC = "moe_layer_fwd_bwd_tokens_per_s"

# DRAM bytes per scatter2scatter launch (ncu: dram__bytes_read.sum + dram__bytes_write.sum, mean of the four launches
# of one layer step). Not measured by this script: it is the figure of the last profiler capture, printed beside
# the live numbers together with where it came from.
NCU_TRAFFIC = {
    "mixtral_8x7b": dict(bytes_per_launch=7.176e9,
                         source="ncu, full size (16384 tokens), the four launches of one timed step of this script "
                                "(up-projection + activation 5.65 GB, down-projection 5.11 GB, down-projection input "
                                "gradient + activation gradient 6.90 GB, up-projection input gradient 11.05 GB; "
                                "algorithmic 4.97 / 2.15 / 4.97 / 4.03 GB), captured at commit 430a1b7"),
}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], tflops_burst=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops_burst=1590.0, tflops_sustained=1400.0, source="fallback")


def load_reference_package():
    """The unmodified reference, installed under baseline/_ref, imported under a name of its own
    (`scattermoe_reference`) so that it can sit beside this repository's `scattermoe` alias package. Importing it
    re-patches the Hugging Face MoE classes (that is what its utils/replace_moe.py does on import); the patches
    that were in place are put back, and the reference's are kept in `PATCHED_FORWARDS` of the returned module."""
    name = "scattermoe_reference"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = os.path.join(ROOT, "baseline", "_ref", "scattermoe")
    init = os.path.join(pkg_dir, "__init__.py")
    if not os.path.exists(init):
        return None
    hf = []
    for modname, cls in (("transformers.models.gpt_oss.modeling_gpt_oss", "GptOssExperts"),
                         ("transformers.models.granitemoehybrid.modeling_granitemoehybrid", "GraniteMoeHybridMoE")):
        try:
            c = getattr(importlib.import_module(modname), cls)
            hf.append((c, c.forward))
        except Exception:
            pass
    spec = importlib.util.spec_from_file_location(name, init, submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    try:
        spec.loader.exec_module(mod)
    except Exception:
        sys.modules.pop(name, None)
        raise
    finally:
        patched = {}
        for c, fwd in hf:
            patched[c.__name__] = c.forward
            c.forward = fwd
        mod.PATCHED_FORWARDS = patched
    return mod


def layer_flops(c, tokens):
    R = tokens * c["k"]
    n1 = 2 * c["F"]
    fwd = 2.0 * R * c["d"] * n1 + 2.0 * R * c["F"] * c["d"]
    return fwd, 3.0 * fwd


def make_routing(cfg_name, T, E, k, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if cfg_name == "granite_zipf":
        pop = torch.arange(1, E + 1, dtype=torch.float32) ** -1.2
        pop = pop / pop.sum()
        logits = logits + torch.log(pop)[torch.randperm(E, generator=g)]
    if cfg_name == "gpt_oss_20b":
        top, idx = torch.topk(logits, k, dim=-1)
        p = torch.softmax(top, dim=-1)
    else:
        p, idx = torch.topk(torch.softmax(logits, dim=-1), k, dim=-1)
        p = p / p.sum(-1, keepdim=True)
    return p, idx


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons (query only). The sampler is started before the warm-up
    (nvidia-smi needs a moment to produce its first line) and only the samples whose timestamp falls inside the
    timed region are kept."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return None
        time.sleep(0.12)                       # let the last in-window sample reach the file
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        import datetime
        sm, mx, reasons, outside = [], [], set(), []
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    clk, cmax = float(f[1]), float(f[2])
                except ValueError:
                    continue
                inside = self.t0 is None or (self.t0 - 0.05 <= ts <= (self.t1 or ts) + 0.05)
                if not inside:
                    outside.append(clk)
                    continue
                sm.append(clk); mx.append(cmax)
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if not sm:
            return {"sm_mhz": statistics.median(outside) if outside else None, "sm_max_mhz": None, "reasons": [],
                    "samples": 0, "note": "timed region shorter than the sampling interval; median of neighbouring samples"}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def build_layer(name, c, tokens, device, seed, ep_world=1, exchange="nvlink", chunks=1, once_per_rank=None):
    """Parameters and inputs of one rank: weights ~N(0, 0.02), X ~N(0, 1), softmax top-k routing."""
    import scattermoe_b200 as sm
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    d, F, E, k = c["d"], c["F"], c["E"], c["k"]

    def rnd(*shape, std):
        out = torch.empty(shape, dtype=bf, device=device)
        # generate on the device in slabs: the CPU generator would take minutes for multi-GB tensors
        gd = torch.Generator(device=device).manual_seed(seed + sum(shape))
        out.normal_(0.0, std, generator=gd)
        return out

    layer = {}
    if c["kind"] == "gpt_oss":
        layer["w1"] = rnd(E, d, 2 * F, std=0.02).requires_grad_()     # (E, in, out) as gpt-oss stores it
        layer["w2"] = rnd(E, F, d, std=0.02).requires_grad_()
        layer["b1"] = rnd(E, 2 * F, std=0.02).requires_grad_()
        layer["b2"] = rnd(E, d, std=0.02).requires_grad_()
    elif ep_world > 1:
        from scattermoe_b200.expert_parallel import ExpertParallelGLUMLP, PeerExpertParallelGLUMLP
        if exchange == "nvlink":
            m = PeerExpertParallelGLUMLP(d, F, E, k, global_tokens=tokens * ep_world, chunks=chunks,
                                         once_per_rank=once_per_rank).to(device=device, dtype=bf)
        else:
            m = ExpertParallelGLUMLP(d, F, E, k).to(device=device, dtype=bf)
        with torch.no_grad():
            m.experts.weight.copy_(rnd(E // ep_world, 2 * F, d, std=0.02))
            m.output_experts.weight.copy_(rnd(E // ep_world, d, F, std=0.02))
        layer["module"] = m
    else:
        m = sm.mlp.GLUMLP(d, F, E, k).to(device=device, dtype=bf)
        with torch.no_grad():
            m.experts.weight.copy_(rnd(E, 2 * F, d, std=0.02))
            m.output_experts.weight.copy_(rnd(E, d, F, std=0.02))
        layer["module"] = m
    p, idx = make_routing(name, tokens, E, k, seed)
    host = dict(x=torch.randn(tokens, d, generator=g).to(bf).pin_memory(),
                p=p.to(bf).pin_memory(), idx=idx.pin_memory(),
                dy=torch.randn(tokens, d, generator=g).to(bf).pin_memory())
    return layer, host


def layer_leaves(c, layer):
    if c["kind"] == "gpt_oss":
        return [layer["w1"], layer["w2"], layer["b1"], layer["b2"]]
    m = layer["module"]
    return [m.experts.weight, m.output_experts.weight]


def forward_only(c, layer, x, p, idx):
    import scattermoe_b200 as sm
    if c["kind"] == "gpt_oss":
        from scattermoe_b200 import activation as A
        routing = sm.flatten_sort_count(idx, c["E"])
        return sm.expert_mlp(x, layer["w1"], layer["w2"], p, c["k"], *routing, A.LAYOUT_GPT_OSS, A.ACT_SILU,
                             up_biases=layer["b1"], down_biases=layer["b2"], alpha=1.702, limit=7.0)
    return layer["module"](x, p, idx)


def run_step(c, layer, x, p, idx, dy):
    """One forward + backward through the public API. Returns (y, [dx, dgates, weight / bias gradients ...])."""
    x = x.requires_grad_()
    p = p.requires_grad_()
    y = forward_only(c, layer, x, p, idx)
    grads = torch.autograd.grad(y, [x, p] + layer_leaves(c, layer), dy)
    return y, list(grads)


class LaunchCounter:
    """Counts the kernels this library launches: a proxy in front of the ctypes library that knows how many
    kernels each C entry point enqueues."""
    KERNELS = {"smoe_scatter2scatter_act": 1, "smoe_scatter2scatter_act_bwd": 1, "smoe_ep_dispatch": 1,
               "smoe_ep_return": 1, "smoe_ep_plan_rows": 1, "smoe_scatter2scatter_to_peers": 1, "smoe_ep_barrier": 1, "smoe_sort_count": 3, "smoe_sort_count_static": 3,
               "smoe_offsets_from_sorted": 1, "smoe_scatter2scatter": 1, "smoe_group_bwd_w": 1, "smoe_group": 1,
               "smoe_topk_reduce": 1, "smoe_gate_grad": 1, "smoe_activation_forward": 1, "smoe_activation_backward": 1,
               "smoe_route_topk": 3, "smoe_status_poison": 1, "smoe_gate_grad_from_partials": 1, "smoe_ep_plan_tokens": 1, "smoe_ep_dispatch_meta": 1,
               "smoe_ep_expand": 1, "smoe_ep_combine": 1, "smoe_ep_sum_parts": 1}

    def __init__(self):
        from scattermoe_b200 import _lib
        self._mod, self._real, self.count = _lib, _lib.load(), 0
        self.events = []          # (entry point, start event, end event) on the stream the call enqueued on

    def __getattr__(self, name):
        fn = getattr(self._real, name)
        n = self.KERNELS.get(name, 0)
        if not n:
            return fn

        def counted(*a):
            self.count += n
            if name == "smoe_group_bwd_w" and a[14]:      # a bias gradient adds its own column-sum kernel
                self.count += 1
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            rc = fn(*a)
            s1.record()
            if rc == self._mod.SMOE_ERR_UNSUPPORTED:      # nothing was launched: the caller takes its two-call form
                self.count -= n
            else:
                self.events.append((name, s0, s1))
            return rc
        return counted

    def ms_by_entry_point(self):
        out = {}
        for name, a, z in self.events:
            out[name] = out.get(name, 0.0) + a.elapsed_time(z)
        return out

    def reset(self):
        self.count, self.events = 0, []

    def install(self):
        self._mod._lib = self

    def remove(self):
        self._mod._lib = self._real


class KernelTimer:
    """CUDA-event brackets around the C-ABI GEMM launches (they run on torch's current stream)."""

    def __init__(self):
        self.records = []   # (kind, flops, start_event, end_event)

    def install(self):
        from scattermoe_b200.kernels import ops
        self._saved = (ops._scatter2scatter_impl, ops._group_bwd_w_impl, ops.scatter2scatter_act,
                       ops._scatter2scatter_act_bwd_impl)
        timer = self
        _s2s, _wg, _s2sa, _s2sb = self._saved

        def bracket():
            return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def s2sa(X, W, se, ss, k, *a, **kw):
            e0, e1 = bracket()
            e0.record()
            res = _s2sa(X, W, se, ss, k, *a, **kw)
            e1.record()
            if res is not None:
                timer.records.append(("scatter2scatter", 2.0 * se.numel() * X.size(1) * W.size(-1), e0, e1))
            return res

        def s2sb(d_up, DY, W, up, *a):
            e0, e1 = bracket()
            e0.record()
            ok = _s2sb(d_up, DY, W, up, *a)
            e1.record()
            if ok:
                timer.records.append(("scatter2scatter", 2.0 * DY.size(0) * DY.size(1) * W.size(-1), e0, e1))
            return ok

        def s2s(output, W, X, k, se, ss, b, xg, yg, off):
            e0, e1 = bracket()
            e0.record()
            _s2s(output, W, X, k, se, ss, b, xg, yg, off)
            e1.record()
            timer.records.append(("scatter2scatter", 2.0 * se.numel() * X.size(1) * output.size(1), e0, e1))

        def wg(E, DW, Db, DY, X, off, gi, fan):
            e0, e1 = bracket()
            e0.record()
            _wg(E, DW, Db, DY, X, off, gi, fan)
            e1.record()
            timer.records.append(("group_bwd_w", 2.0 * DY.size(0) * X.size(1) * DY.size(1), e0, e1))
        ops._scatter2scatter_impl, ops._group_bwd_w_impl, ops.scatter2scatter_act = s2s, wg, s2sa
        ops._scatter2scatter_act_bwd_impl = s2sb

    def remove(self):
        from scattermoe_b200.kernels import ops
        (ops._scatter2scatter_impl, ops._group_bwd_w_impl, ops.scatter2scatter_act,
         ops._scatter2scatter_act_bwd_impl) = self._saved

    def summary(self):
        out = {}
        for kind, flops, a, z in self.records:
            d = out.setdefault(kind, dict(launches=0, ms=0.0, flops=0.0))
            d["launches"] += 1
            d["ms"] += a.elapsed_time(z)
            d["flops"] += flops
        return out


# ---- the reference's own Triton kernels on the same GPU ------------------------------------------------------

class TritonReference:
    """The unmodified reference from baseline/_ref through its own public API (`GLUMLP`, or the call sequence of its
    patched GptOssExperts.forward, utils/replace_moe.py:22-55), with THIS benchmark's weights and inputs."""

    def __init__(self, name, c, layer, host, device):
        self.ref = load_reference_package()
        if self.ref is None:
            raise RuntimeError("baseline/_ref holds no installed copy of the reference")
        ref, bf = self.ref, torch.bfloat16
        d, F, E, k = c["d"], c["F"], c["E"], c["k"]
        self.c = c
        self.x, self.p, self.idx, self.dy = (host[n].to(device) for n in ("x", "p", "idx", "dy"))
        idx = self.idx
        if c["kind"] == "gpt_oss":
            w1, w2, b1, b2 = (layer[n].detach().clone().requires_grad_() for n in ("w1", "w2", "b1", "b2"))
            self.leaves = [w1, w2, b1, b2]

            def fwd(xx, pp):
                routing = ref.flatten_sort_count(idx.flatten(), num_experts=E)
                gu = ref.parallel_linear(xx, w1, k, *routing, expert_biases=b1, grouped_in=False, grouped_out=True)
                gate, up = gu[..., ::2], gu[..., 1::2]
                gate = gate.clamp(min=None, max=7.0)
                up = up.clamp(min=-7.0, max=7.0)
                h = (up + 1) * (gate * torch.sigmoid(gate * 1.702))
                return ref.parallel_linear(h, w2, 1, *routing, expert_biases=b2, grouped_in=True, grouped_out=False,
                                           gates=pp)
        else:
            m = ref.mlp.GLUMLP(d, F, E, k).to(device=device, dtype=bf)
            with torch.no_grad():
                m.experts.weight.copy_(layer["module"].experts.weight)
                m.output_experts.weight.copy_(layer["module"].output_experts.weight)
            self.leaves = [m.experts.weight, m.output_experts.weight]

            def fwd(xx, pp):
                return m(xx, pp, idx)
        self.fwd = fwd

    def forward(self):
        return self.fwd(self.x.detach().requires_grad_(), self.p.detach().requires_grad_())

    def step(self):
        xx, pp = self.x.detach().requires_grad_(), self.p.detach().requires_grad_()
        y = self.fwd(xx, pp)
        return y, list(torch.autograd.grad(y, [xx, pp] + self.leaves, self.dy))

    def routing(self):
        return self.ref.flatten_sort_count(self.idx.flatten(), num_experts=self.c["E"])

    def time(self, iters=5, warmup=3):
        out = {}
        def inference():
            with torch.no_grad():
                return self.fwd(self.x, self.p)
        for key, fn in (("ms_per_step", self.step), ("forward_ms", self.forward), ("inference_ms", inference)):
            for _ in range(warmup):
                fn()
            torch.cuda.synchronize()
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(iters):
                fn()
            z.record()
            torch.cuda.synchronize()
            out[key] = a.elapsed_time(z) / iters
        T = self.x.size(0)
        return {"impl": "reference Triton kernels (unmodified, baseline/_ref), same GPU, same weights and inputs",
                "ms_per_step": out["ms_per_step"], "value": T / (out["ms_per_step"] / 1e3), "unit": "tokens/s",
                "forward_ms": out["forward_ms"], "forward_value": T / (out["forward_ms"] / 1e3),
                "inference_ms": out["inference_ms"], "iters": iters}


# ---- parity, outside the timed regions ------------------------------------------------------------------------

RTOL, ATOL = 2e-2, 2e-2          # the bf16 contract: outputs and gradients against the reference's own kernels
MISMATCH_BUDGET = 1e-4           # fraction of elements allowed outside it (two bf16 runs that round intermediates at
#                                  different places disagree by one bf16 step on a few elements next to zero)


def _compare(got, want, scale=None):
    """|got - want| <= ATOL + RTOL * |want| elementwise, in units of `scale`.

    Every quantity here is a sum of many bf16-rounded terms, so two correct bf16 runs differ by an ABSOLUTE error
    proportional to the typical size of the sum (about 2^-8 of its rms per rounding step), whatever the size of the
    individual element. The absolute tolerance is therefore applied in units of the quantity's rms where that
    exceeds 1 (`scale` None), or of the stated scale (a tensor or number: the square root of the length of the
    sum for weight and bias gradients, whose size differs from expert to expert). `unscaled_mismatch_frac` is the
    same test with no scale at all."""
    got, want = got.detach().float(), want.detach().float()
    raw = (got - want).abs()
    unscaled = float((raw > (ATOL + RTOL * want.abs())).sum().item()) / max(raw.numel(), 1)
    if scale is None:
        scale = max(1.0, float(want.pow(2).mean().sqrt().item())) if want.numel() else 1.0
        used = scale
    else:
        used = "per expert"
    got, want = got / scale, want / scale
    diff = (got - want).abs()
    bad = diff > (ATOL + RTOL * want.abs())
    frac = float(bad.sum().item()) / max(diff.numel(), 1)
    return {"max_abs": float(raw.max().item()) if raw.numel() else 0.0, "mismatch_frac": frac,
            "unscaled_mismatch_frac": unscaled, "scale": used,
            "ok": bool(frac <= MISMATCH_BUDGET and bool(torch.isfinite(got).all()))}


def dense_loop_rows(c, layer, x, p, idx, dy, rows):
    """fp32 dense per-expert loop (plain PyTorch, TF32 off) for a sample of token rows: y, dx, dgates of those rows.
    Every quantity of a token depends on that token and the weights alone, so a row sample checks the full-size
    run. Restates the reference test's ground truth (tests/test_mlp.py:10-26) per expert."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        xs = x[rows].float().requires_grad_()
        ps = p[rows].float().requires_grad_()
        ids = idx[rows]
        F = c["F"]
        y = torch.zeros_like(xs)
        for e in ids.unique().tolist():
            tok, slot = (ids == e).nonzero(as_tuple=True)
            if c["kind"] == "gpt_oss":
                w1, w2 = layer["w1"][e].detach().float(), layer["w2"][e].detach().float()          # (in, out)
                up = xs[tok] @ w1 + layer["b1"][e].detach().float()
                gate, lin = up[:, ::2].clamp(max=7.0), up[:, 1::2].clamp(-7.0, 7.0)
                h = (lin + 1) * (gate * torch.sigmoid(gate * 1.702))
                out = h @ w2 + layer["b2"][e].detach().float()
            else:
                m = layer["module"]
                up = xs[tok] @ m.experts.weight[e].detach().float().t()
                h = torch.nn.functional.silu(up[:, F:]) * up[:, :F]              # second half activated (mlp.py:81-87)
                out = h @ m.output_experts.weight[e].detach().float().t()
            y = y.index_add(0, tok, out * ps[tok, slot].unsqueeze(1))
        dx, dp = torch.autograd.grad(y, [xs, ps], dy[rows].float())
        return y.detach(), dx, dp
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def parity_check(name, c, layer, dev_in, triton_ref, sample_rows=256):
    """One more full-size step of this library, compared with (a) the reference's Triton kernels on the same
    weights and inputs and (b) the fp32 dense loop on a sample of token rows."""
    import scattermoe_b200 as sm
    out = {"rtol": RTOL, "atol": ATOL, "mismatch_budget": MISMATCH_BUDGET}
    x, p, idx, dy = dev_in["x"], dev_in["p"], dev_in["idx"], dev_in["dy"]
    y, grads = run_step(c, layer, x.detach(), p.detach(), idx, dy)
    sm.check_device_status(x.device)
    T, d, E = x.size(0), c["d"], c["E"]
    root_rows = torch.bincount(idx.flatten(), minlength=E).clamp(min=1).float().sqrt()
    names = ["dx", "dgates", "dw1", "dw2", "db1", "db2"][:len(grads)]
    ok = True
    if triton_ref is not None:
        se, ss, off = sm.flatten_sort_count(idx, E)
        rse, rss, roff = triton_ref.routing()
        routing = {"sorted_expert_idxs_equal": bool(torch.equal(se, rse)),
                   "expert_offsets_equal": bool(torch.equal(off, roff)),
                   "sorted_scattered_idxs_equal": bool(torch.equal(ss, rss))}
        if not routing["sorted_scattered_idxs_equal"]:
            # torch.sort without stable=True may order ties differently: then the orders must agree per expert as sets
            same, start = True, 0
            for end in off.tolist():
                same = same and torch.equal(torch.sort(ss[start:end]).values, torch.sort(rss[start:end]).values)
                start = end
            routing["sorted_scattered_idxs_equal_per_expert_as_sets"] = bool(same)
            ok = ok and same
        ok = ok and routing["sorted_expert_idxs_equal"] and routing["expert_offsets_equal"]
        ry, rgrads = triton_ref.step()
        q = {"y": _compare(y, ry)}
        for n, g, rg in zip(names, grads, rgrads):
            scale = None
            if n in ("dw1", "dw2"):
                scale = root_rows.view(E, 1, 1)               # sums over the expert's rows
            elif n in ("db1", "db2"):
                scale = root_rows.view(E, 1)
            if n in ("dw1", "dw2") and g.numel() > (1 << 28):
                # a sample of (expert, row-band) blocks of the big weight gradients keeps the check cheap
                sel = torch.arange(0, g.size(1), max(1, g.size(1) // 64), device=g.device)
                q[n] = _compare(g[:, sel], rg[:, sel], scale)
                q[n]["sampled_rows_per_expert"] = int(sel.numel())
            else:
                q[n] = _compare(g, rg, scale)
        out["vs_reference_gpu"] = {"ok": all(v["ok"] for v in q.values()), "quantities": q, "routing": routing,
                                   "scales": "y, dx, dgates in units of max(1, rms of the reference's tensor); dw, db "
                                             "divided by sqrt(rows of the expert): sums of n bf16-rounded products "
                                             "differ between two correct bf16 runs by about 2^-8 * sqrt(n) * "
                                             "rms(term), whatever the size of the element"}
        ok = ok and out["vs_reference_gpu"]["ok"]
        del ry, rgrads
    else:
        out["vs_reference_gpu"] = None
    # (b) fp32 dense loop on sampled token rows
    g = torch.Generator().manual_seed(1)
    rows = torch.randperm(T, generator=g)[:min(sample_rows, T)].to(x.device)
    ty, tdx, tdp = dense_loop_rows(c, layer, x, p, idx, dy, rows)

    def rms(a, b):
        return float((a.float() - b).pow(2).mean().sqrt().item())
    ours = {"y": rms(y[rows], ty), "dx": rms(grads[0][rows], tdx), "dgates": rms(grads[1][rows], tdp)}
    dl = {"tokens": int(rows.numel()), "ours_rms_err": ours,
          "truth_rms": {"y": float(ty.pow(2).mean().sqrt()), "dx": float(tdx.pow(2).mean().sqrt()),
                        "dgates": float(tdp.pow(2).mean().sqrt())}}
    # an rms error within 2 % (the contract's rtol) of the rms of the quantity passes
    dl["ok"] = all(ours[n] <= RTOL * dl["truth_rms"][n] + 1e-6 for n in ours)
    if triton_ref is not None:
        ry, rgrads = triton_ref.step()
        dl["reference_rms_err"] = {"y": rms(ry[rows], ty), "dx": rms(rgrads[0][rows], tdx),
                                   "dgates": rms(rgrads[1][rows], tdp)}
        del ry, rgrads
    out["vs_dense_loop"] = dl
    ok = ok and dl["ok"]
    mx = [v["max_abs"] for v in (out["vs_reference_gpu"] or {}).get("quantities", {}).values()]
    out["max_abs"] = max(mx) if mx else None
    out["ok"] = bool(ok)
    del y, grads
    torch.cuda.empty_cache()
    return out


def ep_parity_check(device, rank, world, dist, exchange, chunks, once_per_rank=None):
    """N > 1: one small seeded expert-parallel step; every rank compares its outputs and gradient slices with the
    single-GPU layer on the gathered problem (same seed on every rank, so nothing needs gathering)."""
    import scattermoe_b200 as sm
    from scattermoe_b200.expert_parallel import ExpertParallelGLUMLP, PeerExpertParallelGLUMLP
    T, d, F, E, k = 1024 * world, 512, 256, 8 * world, 4
    g = torch.Generator().manual_seed(123)
    bf = torch.bfloat16
    x = torch.randn(T, d, generator=g).to(bf).to(device)
    p, idx = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), k)
    p = (p / p.sum(-1, keepdim=True)).to(bf).to(device)
    idx = idx.to(device)
    w1 = (torch.randn(E, 2 * F, d, generator=g) * 0.05).to(bf).to(device)
    w2 = (torch.randn(E, d, F, generator=g) * 0.05).to(bf).to(device)
    dy = torch.randn(T, d, generator=g).to(bf).to(device)
    single = sm.mlp.GLUMLP(d, F, E, k).to(device=device, dtype=bf)
    with torch.no_grad():
        single.experts.weight.copy_(w1)
        single.output_experts.weight.copy_(w2)
    xs, ps = x.clone().requires_grad_(), p.clone().requires_grad_()
    want_y = single(xs, ps, idx)
    want = [want_y] + list(torch.autograd.grad(want_y, [xs, ps, single.experts.weight, single.output_experts.weight], dy))
    tl, el = T // world, E // world
    ts, es = slice(rank * tl, (rank + 1) * tl), slice(rank * el, (rank + 1) * el)
    if exchange == "nvlink":
        m = PeerExpertParallelGLUMLP(d, F, E, k, chunks=chunks, once_per_rank=once_per_rank).to(device=device, dtype=bf)
    else:
        m = ExpertParallelGLUMLP(d, F, E, k).to(device=device, dtype=bf)
    with torch.no_grad():
        m.experts.weight.copy_(w1[es])
        m.output_experts.weight.copy_(w2[es])
    xx, pp = x[ts].clone().requires_grad_(), p[ts].clone().requires_grad_()
    for _ in range(2):
        y = m(xx, pp, idx[ts])
        got = [y] + list(torch.autograd.grad(y, [xx, pp, m.experts.weight, m.output_experts.weight], dy[ts]))
    sm.check_device_status(device)
    rows = torch.bincount(idx.flatten(), minlength=E).clamp(min=1).float().sqrt().to(device)
    res = {"y": _compare(got[0], want[0][ts]), "dx": _compare(got[1], want[1][ts]),
           "dgates": _compare(got[2], want[2][ts]),
           "dw1": _compare(got[3], want[3][es], rows[es].view(-1, 1, 1)),
           "dw2": _compare(got[4], want[4][es], rows[es].view(-1, 1, 1))}
    worst = torch.tensor([max(v["max_abs"] for v in res.values()), 0.0 if all(v["ok"] for v in res.values()) else 1.0],
                         device=device)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    del m
    torch.cuda.empty_cache()
    return {"against": "single-GPU GLUMLP of this library on the gathered problem (T=%d, d=%d, F=%d, E=%d, k=%d)"
                       % (T, d, F, E, k), "max_err": float(worst[0].item()), "ok": bool(worst[1].item() == 0.0),
            "rtol": RTOL, "atol": ATOL, "rank0": res}


# ---- the reference's CPU path ---------------------------------------------------------------------------------

def cpu_reference(name, c, steps, warmup, budget_s=None):
    """Dense per-expert fp32 loop on all host cores, `steps` timed steps after `warmup` on a token sample. With a
    time budget the sample shrinks (after a first probing step) so that the whole run ends within it."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import scattermoe_oracle as oracle
    tokens = min(CPU_SAMPLE_TOKENS.get(name, 1024), c["T"])
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = name if name in oracle.CONFIGS else "tiny_fp32_gelu"
    b = oracle.DenseLoopBench(cfg, tokens, threads=cores)
    probe = b.step()
    if budget_s is not None and probe * (steps + warmup) > budget_s and tokens > 256:
        tokens = max(256, int(tokens * budget_s / (probe * (steps + warmup))) // 256 * 256)
        b = oracle.DenseLoopBench(cfg, tokens, threads=cores)
    threads = b.threads
    times = []
    for i in range(warmup + steps):
        t = b.step()
        if i >= warmup:
            times.append(t)
    sec = sum(times) / len(times)
    return dict(value=tokens / sec, unit="tokens/s", cores=threads, kind="port",
                sample="%d of %d tokens per step, fp32 dense per-expert loop, forward+backward, %.2f s/step, %d timed "
                       "steps" % (tokens, c["T"], sec, len(times))), sec, tokens


# ---- one workload on this process's GPU -----------------------------------------------------------------------

def measure(name, c, device, rank, world, dist, steps, warmup, with_e2e=True, sampler_gpu=None, exchange="nvlink",
            chunks=1, keep=False, once_per_rank=None):
    """Device-timed forward+backward (and forward, and end-to-end) of one workload. Returns (fields, state)."""
    import scattermoe_b200 as sm
    peaks = load_peaks()
    ep = world > 1 and c["kind"] != "gpt_oss"
    tokens_local = c["T"] // world if ep else c["T"]
    tokens_all = c["T"] if ep else c["T"] * world
    layer, host = build_layer(name, c, tokens_local, device, seed=rank, ep_world=world if ep else 1, exchange=exchange,
                             chunks=chunks, once_per_rank=once_per_rank)
    dev_in = {n: t.to(device) for n, t in host.items()}

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def resident_step():
        return run_step(c, layer, dev_in["x"].detach(), dev_in["p"].detach(), dev_in["idx"], dev_in["dy"])

    def forward_step():
        return forward_only(c, layer, dev_in["x"].detach().requires_grad_(), dev_in["p"].detach().requires_grad_(),
                            dev_in["idx"])

    out_host = dict(y=torch.empty_like(host["x"]).pin_memory(), dx=torch.empty_like(host["x"]).pin_memory())
    # two copy streams, one per direction: PCIe is full duplex, and a result travelling back must not queue behind the
    # next step's inputs
    copy_stream = torch.cuda.Stream(device=device)
    back_stream = torch.cuda.Stream(device=device) if COPY_STREAMS == 2 else copy_stream
    staged = {}

    def stage_inputs():
        """Enqueue the host->device copies of one step's inputs on the copy stream."""
        with torch.cuda.stream(copy_stream):
            staged["in"] = {n: host[n].to(device, non_blocking=True) for n in ("x", "p", "idx", "dy")}
            staged["ready"] = torch.cuda.Event()
            staged["ready"].record(copy_stream)

    pending = []      # (y, dx, copied event) of the steps whose results may still be travelling to the host

    def e2e_step(prefetch):
        # Every step copies its own inputs from pinned host memory and its results back. The copies run on two
        # streams of their own: the next step's inputs are enqueued while this step computes, and this step's
        # results travel back while the next step computes.
        cur = torch.cuda.current_stream(device)
        # results older than the previous step's: their copies ended long ago; after this wait their memory may be
        # reused by what this step enqueues (the tensors are allocated on `cur`, only read on `back_stream`)
        while len(pending) > 1:
            cur.wait_event(pending.pop(0)[2])
        cur.wait_event(staged["ready"])
        ins = staged.pop("in")
        for t in ins.values():
            t.record_stream(cur)
        if prefetch:
            stage_inputs()
        y, grads = run_step(c, layer, ins["x"], ins["p"], ins["idx"], ins["dy"])
        dx = grads[0]
        done = torch.cuda.Event()
        done.record(cur)
        copied = torch.cuda.Event()
        with torch.cuda.stream(back_stream):
            back_stream.wait_event(done)
            out_host["y"].copy_(y, non_blocking=True)
            out_host["dx"].copy_(dx, non_blocking=True)
            copied.record(back_stream)
        pending.append((y, dx, copied))

    def e2e_loop(n):
        # Nothing is staged before the loop starts (the first step's host->device copy is not hidden) and the
        # last step's device->host copy is joined before it ends: every copy lies inside the timed bracket.
        staged.clear()
        stage_inputs()
        for i in range(n):
            e2e_step(prefetch=(i + 1 < n))
        torch.cuda.current_stream(device).wait_stream(copy_stream)
        torch.cuda.current_stream(device).wait_stream(back_stream)
        pending.clear()

    def timed(fn, n):
        # No cyclic garbage collection inside a timed region: a collection that happens to free an earlier
        # workload's peer-mapped buffers unmaps them on every rank and stalls this one for hundreds of milliseconds
        # (seen as a 50 ms/step outlier in a 6-step end-to-end loop).
        gc.collect()
        gc.disable()
        try:
            barrier()
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn(n)
            z.record()
            barrier()
        finally:
            gc.enable()
        ms = a.elapsed_time(z)
        if dist is not None:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    def loop(fn):
        def run(n):
            for _ in range(n):
                fn()
        return run

    sampler = ClockSampler(sampler_gpu) if (rank == 0 and sampler_gpu is not None) else None
    if sampler:
        sampler.start()
    for _ in range(warmup):
        resident_step()
    sm.check_device_status(device)
    timer = KernelTimer()
    timer.install()
    counter = LaunchCounter()
    counter.install()
    BAD = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"}
    remeasured = False
    clocks = None
    try:
        while True:
            if sampler:
                sampler.mark_begin()
            ms_total = timed(loop(resident_step), steps)
            if sampler:
                sampler.mark_end()
            clocks = sampler.stop() if sampler else None
            bad = bool(clocks and BAD & set(clocks.get("reasons", [])))
            if world > 1:      # every rank must take the same decision
                flag = torch.tensor([1 if bad else 0], device=device)
                dist.broadcast(flag, src=0)
                bad = bool(flag.item())
            if not bad or remeasured or sampler_gpu is None:
                break
            # a thermal / hardware slowdown was active during the timed region: the number is rejected and taken once more
            remeasured = True
            timer.records.clear()
            counter.reset()
            if rank == 0:
                sampler = ClockSampler(sampler_gpu)
                sampler.start()
                time.sleep(0.3)
        if clocks is not None:
            clocks["remeasured_after_slowdown"] = remeasured
        launches = counter.count
        abi_ms = {k_: round(v_ / steps, 4) for k_, v_ in sorted(counter.ms_by_entry_point().items())}
    finally:
        counter.remove()
        timer.remove()
    ksum = timer.summary()
    mod = layer.get("module")
    if hasattr(mod, "live_row_fraction"):
        # peer-memory expert parallelism launches its GEMMs over worst-case-sized buffers; count the live rows only
        live = mod.live_row_fraction()
        for d_ in ksum.values():
            d_["flops"] *= live
    tensor_core = sm.kernels.ops.last_path_was_tensor_core()

    for _ in range(2):
        forward_step()
    ms_fwd = timed(loop(forward_step), steps)

    def inference_step():
        with torch.no_grad():
            return forward_only(c, layer, dev_in["x"], dev_in["p"], dev_in["idx"])
    for _ in range(2):
        inference_step()
    ms_inf = timed(loop(inference_step), steps)

    ms_e2e = None
    if with_e2e:
        e2e_loop(4)          # the caching allocator reaches its steady state (no cudaMalloc inside the timed loop)
        ms_e2e = timed(e2e_loop, steps)
    sm.check_device_status(device)

    ms_step = ms_total / steps
    fwd_flops, fb_flops = layer_flops(c, tokens_all)
    peak = peaks["tflops_sustained"]
    dom = ksum.get("scatter2scatter", dict(launches=0, ms=0.0, flops=0.0))
    achieved = dom["flops"] / (dom["ms"] / 1e3) / 1e12 if dom["ms"] > 0 else 0.0
    traffic = NCU_TRAFFIC.get(name) if world == 1 else None
    roofline = {"bound": "tensor",
                "kernel": "s2s_tc_kernel (scatter2scatter: 2 forward + 2 input-gradient launches per step)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": "%s, sustained bf16 (kernel timed inside a long step)" % peaks["source"],
                "launches": dom["launches"], "avg_launch_ms": dom["ms"] / max(dom["launches"], 1),
                "traffic": traffic["bytes_per_launch"] if traffic else None,
                "traffic_source": traffic["source"] if traffic else None}
    wg = ksum.get("group_bwd_w")
    if wg and wg["ms"] > 0:
        roofline["group_bwd_w"] = {"achieved": wg["flops"] / (wg["ms"] / 1e3) / 1e12, "launches": wg["launches"],
                                   "avg_launch_ms": wg["ms"] / wg["launches"],
                                   "frac": wg["flops"] / (wg["ms"] / 1e3) / 1e12 / peak}
    fields = {
        "value": tokens_all / (ms_step / 1e3), "ms_per_step": ms_step,
        "layer_tflops": fb_flops / (ms_step / 1e3) / 1e12,
        "layer_frac_of_bf16_peak": fb_flops / world / (ms_step / 1e3) / 1e12 / peak,
        "tensor_core_path": bool(tensor_core),
        "roofline": roofline,
        "forward": {"value": tokens_all / (ms_fwd / steps / 1e3), "unit": "tokens/s", "ms_per_step": ms_fwd / steps,
                    "frac_of_bf16_peak": fwd_flops / world / (ms_fwd / steps / 1e3) / 1e12 / peak,
                    "what": "the training forward alone (autograd on, tensors for backward saved)",
                    "inference_ms_per_step": ms_inf / steps,
                    "inference_value": tokens_all / (ms_inf / steps / 1e3),
                    "inference_what": "the same forward under torch.no_grad (nothing kept for backward)"},
        # kernels of this library launched by this rank inside the timed region (counted at the C-ABI boundary)
        "gpu_launches": launches,
        # device time between the events bracketing each C-ABI call, summed over the timed region, per step
        "abi_ms_per_step": abi_ms,
        "clocks": clocks,
    }
    if ms_e2e is not None:
        h2d = sum(host[n].numel() * host[n].element_size() for n in ("x", "p", "idx", "dy"))
        d2h = sum(t.numel() * t.element_size() for t in out_host.values())
        fields["e2e"] = {"value": tokens_all / (ms_e2e / steps / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                         "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / steps}
    staged.clear()
    state = dict(tokens_all=tokens_all, tokens_local=tokens_local, ep=ep)
    if keep:
        state.update(layer=layer, host=host, dev_in=dev_in)
    else:
        del layer, host, dev_in, out_host
        torch.cuda.empty_cache()
    return fields, state


COPY_STREAMS = 2      # end-to-end loop: one copy stream per direction (2) or one for both (1); see --copy-streams


def describe(name, c, world, ep, exchange, tokens_all, tokens_local):
    return {"workload": name, "global_tokens": tokens_all, "tokens_per_gpu": tokens_local, "d_model": c["d"],
            "d_ffn": c["F"], "experts": c["E"], "experts_per_gpu": c["E"] // world if ep else c["E"],
            "top_k": c["k"], "activation": c["kind"], "bias": c["bias"],
            "parallelism": ("ep%d: experts partitioned, %s dispatch/combine"
                            % (world, "NVLink peer-memory" if exchange == "nvlink" else "NCCL all-to-all-v")) if ep
            else ("single GPU" if world == 1 else "replicas on token shards"),
            "l2": "weights and activations exceed L2 (126 MB) every step"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="mixtral_8x7b", choices=sorted(LAYERS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--exchange", default="nvlink", choices=["nvlink", "nccl"],
                    help="expert-parallel row exchange for N > 1: peer-memory kernels over NVLink, or NCCL all-to-all-v")
    ap.add_argument("--chunks", type=int, default=1,
                    help="pipeline chunks of the NVLink exchange (each chunk's transfers overlap the other's GEMMs)")
    ap.add_argument("--once-per-rank", choices=("auto", "on", "off"), default="auto",
                    help="NVLink exchange: send each token once per owning rank instead of once per slot (auto: when "
                         "that saves at least 70 % of the rows)")
    ap.add_argument("--separate-return", action="store_true",
                    help="per-slot NVLink exchange: return rows with a push kernel after the GEMM instead of from the "
                         "GEMM's own epilogue")
    ap.add_argument("--copy-streams", type=int, choices=(1, 2), default=COPY_STREAMS,
                    help="end-to-end loop: host->device and device->host copies on one stream each, or both on one")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-triton-ref", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="skip the short measurements of the other workloads (other_configs / ep_config5)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    name, c = args.config, LAYERS[args.config]
    ep = world > 1 and c["kind"] != "gpt_oss"
    if ep and (c["E"] % world or c["T"] % world):
        raise SystemExit("expert parallel needs the world size to divide E=%d and T=%d" % (c["E"], c["T"]))
    scaling = "weak" if (world > 1 and not ep) else "strong"

    if args.impl == "reference":
        if rank != 0:
            return
        steps, warmup = max(1, args.steps), max(0, args.warmup)
        base, sec, sample = cpu_reference(name, c, steps, warmup, budget_s=CPU_ARM_BUDGET_S)
        tokens_local = c["T"] // world if ep else c["T"]
        tokens_all = c["T"] if ep else c["T"] * world
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
                "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": describe(name, c, world, ep, args.exchange, tokens_all, tokens_local),
                "sampled": sample < c["T"], "sample_tokens": sample, "full_tokens": c["T"],
                "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU path); use --impl reference for the CPU baseline")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    once = {"auto": None, "on": True, "off": False}[args.once_per_rank]
    globals()["COPY_STREAMS"] = args.copy_streams
    if args.separate_return:
        import scattermoe_b200.expert_parallel as _ep
        _ep.FUSE_RETURN = False
    fields, st = measure(name, c, device, rank, world, dist, args.steps, args.warmup, with_e2e=True,
                         sampler_gpu=local_rank, exchange=args.exchange, chunks=args.chunks, keep=(world == 1),
                         once_per_rank=once)
    line = {"metric": METRIC, "value": fields.pop("value"), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": fields.pop("ms_per_step"), "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": describe(name, c, world, st["ep"], args.exchange, st["tokens_all"], st["tokens_local"])}
    line.update(fields)
    failed = False

    if world == 1:
        triton_ref = None
        if not args.no_triton_ref:
            try:
                triton_ref = TritonReference(name, c, st["layer"], st["host"], device)
                line["reference_gpu"] = triton_ref.time()
            except Exception as e:  # the comparison is informative; it must not break the benchmark line
                triton_ref = None
                line["reference_gpu"] = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
        if not args.no_parity:
            line["parity"] = parity_check(name, c, st["layer"], st["dev_in"], triton_ref)
            failed = failed or not line["parity"]["ok"]
        del triton_ref
        st.clear()
        torch.cuda.empty_cache()
    elif not args.no_parity and ep:
        line["parity"] = ep_parity_check(device, rank, world, dist, args.exchange, args.chunks, once)
        failed = failed or not line["parity"]["ok"]

    if not args.no_other_configs and name == "mixtral_8x7b":
        # the remaining workloads, short runs, so that the record of this run holds them too
        short_steps, short_warm = min(args.steps, 6), 3
        others = {}
        for other in (("gpt_oss_20b", "granite_zipf", "qwen3_moe_ep") if world == 1 else ("qwen3_moe_ep",)):
            oc = LAYERS[other]
            if world > 1 and (oc["E"] % world or oc["T"] % world):
                continue
            try:
                f, ost = measure(other, oc, device, rank, world, dist, short_steps, short_warm, with_e2e=(world > 1),
                                 sampler_gpu=None, exchange=args.exchange, chunks=args.chunks, keep=(world == 1),
                                 once_per_rank=once)
                entry = {"ms_per_step": f["ms_per_step"], "value": f["value"], "unit": "tokens/s", "steps": short_steps,
                         "warmup": short_warm, "layer_frac_of_bf16_peak": f["layer_frac_of_bf16_peak"],
                         "forward_ms": f["forward"]["ms_per_step"], "abi_ms_per_step": f["abi_ms_per_step"],
                         "roofline_frac": f["roofline"]["frac"],
                         "config": describe(other, oc, world, ost["ep"], args.exchange, ost["tokens_all"],
                                            ost["tokens_local"])}
                if "e2e" in f:
                    entry["e2e"] = f["e2e"]
                if world == 1:
                    if not args.no_triton_ref:
                        try:
                            tr = TritonReference(other, oc, ost["layer"], ost["host"], device)
                            entry["reference_gpu"] = tr.time(iters=3, warmup=2)
                            if not args.no_parity:
                                entry["parity"] = parity_check(other, oc, ost["layer"], ost["dev_in"], tr)
                                failed = failed or not entry["parity"]["ok"]
                            del tr
                        except Exception as e:
                            entry["reference_gpu"] = {"unavailable": "%s: %s" % (type(e).__name__, str(e)[:200])}
                    ost.clear()
                    torch.cuda.empty_cache()
                others[other] = entry
            except Exception as e:
                others[other] = {"failed": "%s: %s" % (type(e).__name__, str(e)[:300])}
                failed = True
        if "qwen3_moe_ep" in others:
            # BASELINE config 5 at this N (the single-GPU layer at N = 1): the expert-parallel scaling curve
            line["ep_config5"] = others.pop("qwen3_moe_ep")
        if others:
            line["other_configs"] = others

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"], _, _ = cpu_reference(name, c, 1, 0)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    if failed:
        print("bench.py: a parity check failed (see the `parity` keys of the line above)", file=sys.stderr)
        sys.exit(3)


if __name__ == "__main__":
    main()
