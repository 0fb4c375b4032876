"""Single-launch timings of the grouped-GEMM kernels at a named layer shape.

    python kernel_bench.py --workload mixtral_8x7b --launch all

times, with CUDA events around back-to-back launches on torch's current stream, the launches one layer step makes
through `kernels.ops` (rows already in expert order, as `parallel_linear` feeds them): the up-projection with and
without the fused activation, the down-projection, the two input gradients (the down-projection's also with the
fused activation gradient) and the two weight gradients, plus the down-projection in the form that stores its rows
into peer buffers (`gemm2_to_peers`, with this GPU as the only peer). One JSON line per measurement. `--tokens` shrinks the problem (for profiler captures); the weights keep the workload's shape.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

WORKLOADS = {   # tokens, d_model, d_ffn, experts, top_k
    "mixtral_8x7b": (16384, 4096, 14336, 8, 2),
    "gpt_oss_20b": (8192, 2880, 2880, 32, 4),
    "qwen3_moe": (8192, 2048, 768, 128, 8),
}
LAUNCHES = ("gemm1", "gemm1_act", "gemm2", "gemm2_to_peers", "dgrad2", "dgrad2_act", "dgrad1", "wgrad1", "wgrad2")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="mixtral_8x7b")
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--launch", default="all", help="'all' or a comma-separated list of: " + ", ".join(LAUNCHES))
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args(argv)

    import scattermoe_b200 as sm
    from scattermoe_b200 import activation as act
    from scattermoe_b200.kernels import ops

    T, d, F, E, k = WORKLOADS[a.workload]
    T = a.tokens or T
    dev, dt = "cuda", torch.bfloat16
    torch.manual_seed(0)
    se, ss, off = sm.flatten_sort_count(torch.topk(torch.randn(T, E, device=dev), k).indices, E)
    R = T * k
    x = torch.randn(R, d, device=dev, dtype=dt)            # token rows in expert order
    h = torch.randn(R, F, device=dev, dtype=dt)            # hidden rows
    d_up = torch.randn(R, 2 * F, device=dev, dtype=dt)     # gradient of the up-projection
    w1 = torch.randn(E, 2 * F, d, device=dev, dtype=dt) * 0.02     # nn.Linear storage (E, out, in)
    w2 = torch.randn(E, d, F, device=dev, dtype=dt) * 0.02
    s2s = lambda X, W, yg: ops.scatter2scatter(X, W, se, ss, 1, x_grouped=True, y_grouped=yg, expert_offsets=off)
    # the down-projection whose epilogue returns its rows "home" (expert parallelism): here a world of one whose only
    # peer buffer is local, every row returning to the slot its index names
    import ctypes
    home = torch.empty(R, d, device=dev, dtype=dt)
    home_ptrs = (ctypes.c_void_p * 1)(home.data_ptr())
    calls = {
        "gemm2_to_peers": (lambda: ops.scatter2scatter_to_peers(h, w2.permute(0, 2, 1), off, ss, home_ptrs, d, R, 0, 1),
                           2 * R * d * F),
        "gemm1": (lambda: s2s(x, w1.permute(0, 2, 1), True), 2 * R * d * 2 * F),
        "gemm1_act": (lambda: ops.scatter2scatter_act(x, w1.permute(0, 2, 1), se, ss, 1, act.LAYOUT_GLU_SECOND,
                                                      act.ACT_SILU, x_grouped=True, expert_offsets=off),
                      2 * R * d * 2 * F),
        "gemm2": (lambda: s2s(h, w2.permute(0, 2, 1), False), 2 * R * d * F),
        "dgrad2": (lambda: s2s(x, w2, True), 2 * R * d * F),
        "dgrad2_act": (lambda: ops.scatter2scatter_act_bwd(x, w2, d_up, off, act.LAYOUT_GLU_SECOND, act.ACT_SILU),
                       2 * R * d * F),
        "dgrad1": (lambda: s2s(d_up, w1, False), 2 * R * d * 2 * F),
        "wgrad1": (lambda: ops.group_bwd_W(d_up, x, off, E), 2 * R * d * 2 * F),
        "wgrad2": (lambda: ops.group_bwd_W(x, h, off, E), 2 * R * d * F),
    }
    names = LAUNCHES if a.launch == "all" else tuple(a.launch.split(","))
    for n in names:
        if n not in LAUNCHES:
            ap.error("unknown launch %r" % n)
    ops.FORCE_PATH = "tc"
    try:
        for name in names:
            fn, flop = calls[name]
            for _ in range(a.warmup):
                fn()
            beg, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            beg.record()
            for _ in range(a.iters):
                fn()
            end.record()
            torch.cuda.synchronize()
            sm.check_device_status()
            ms = beg.elapsed_time(end) / a.iters
            print(json.dumps({"workload": a.workload, "tokens": T, "launch": name, "ms": round(ms, 4),
                              "tflops": round(flop / ms / 1e9, 1), "iters": a.iters}), flush=True)
    finally:
        ops.FORCE_PATH = None


if __name__ == "__main__":
    main()
