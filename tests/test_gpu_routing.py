"""Routing bookkeeping on the GPU through the C ABI: bit-exact against the golden vectors and the oracle."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import scattermoe_oracle as oracle  # noqa: E402
from util import golden_names, load_golden, segments_equal_as_sets  # noqa: E402

pytestmark = pytest.mark.gpu


def _run(idx, E):
    import scattermoe_b200 as sm
    se, ss, off = sm.flatten_sort_count(idx.cuda(), num_experts=E)
    torch.cuda.synchronize()
    return se.cpu(), ss.cpu(), off.cpu()


@pytest.mark.parametrize("name", golden_names("sort_"))
def test_sort_golden(name):
    g = load_golden(name)
    se, ss, off = _run(g["expert_idxs"], g["E"])
    assert se.dtype == ss.dtype == off.dtype == torch.int64
    assert torch.equal(se, g["sorted_expert_idxs"])
    assert torch.equal(off, g["expert_offsets"])
    o_se, o_ss, o_off = oracle.flatten_sort_count(g["expert_idxs"], g["E"])
    assert torch.equal(ss, o_ss), "slot order must be the stable one"
    if g["reference_was_stable"]:
        assert torch.equal(ss, g["sorted_scattered_idxs"])
    else:
        assert segments_equal_as_sets(ss, g["sorted_scattered_idxs"], off)


@pytest.mark.parametrize("T,E,k", [(0, 8, 2), (1, 1, 1), (2047, 8, 1), (2048, 8, 1), (2049, 3, 1), (8192, 32, 4),
                                   (32768, 64, 8), (65536, 128, 8), (5000, 1024, 2), (3000, 4096, 3)])
def test_sort_against_oracle(T, E, k):
    g = torch.Generator().manual_seed(T + E + k)
    if T == 0:
        idx = torch.zeros((0, k), dtype=torch.int64)
    else:
        idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(min(T, 64))])
        idx = idx.repeat((T + idx.size(0) - 1) // idx.size(0), 1)[:T]
        idx = idx[torch.randperm(T, generator=g)]
        if E >= 8:
            idx[idx == 3] = 5    # leave expert 3 empty, double expert 5
    se, ss, off = _run(idx, E)
    o_se, o_ss, o_off = oracle.flatten_sort_count(idx, E)
    assert torch.equal(se, o_se) and torch.equal(ss, o_ss) and torch.equal(off, o_off)


def test_sort_properties_at_full_size():
    """Qwen3-MoE-shaped routing (global R = 524288): sortedness, permutation, histogram."""
    from scattermoe_b200.kernels import ops
    p, idx = oracle.make_routing("qwen3_moe_ep", 65536, 128, 8)
    se, ss, off = _run(idx, 128)
    assert bool((se[1:] >= se[:-1]).all())
    assert torch.equal(torch.sort(ss).values, torch.arange(idx.numel()))
    assert torch.equal(idx.flatten()[ss], se)
    assert torch.equal(off, torch.bincount(idx.flatten(), minlength=128).cumsum(0))
    same_e = se[1:] == se[:-1]
    assert bool((ss[1:][same_e] > ss[:-1][same_e]).all()), "stable inside each expert"
    off2 = ops.offsets_from_sorted(se.cuda(), 128).cpu()
    assert torch.equal(off2, off)


def test_int32_ids_keep_their_dtype():
    import scattermoe_b200 as sm
    idx = torch.randint(0, 8, (100, 2), dtype=torch.int32)
    se, ss, off = sm.flatten_sort_count(idx.cuda(), 8)
    assert se.dtype == torch.int32 and ss.dtype == torch.int64 and off.dtype == torch.int64
    assert torch.equal(se.cpu().long(), torch.sort(idx.flatten().long()).values)


def _torch_router(logits, k, mode, renormalize):
    return oracle.route_topk(logits, k, mode, renormalize)


@pytest.mark.parametrize("mode,renorm", [("softmax_topk", True), ("softmax_topk", False), ("topk_softmax", True)])
@pytest.mark.parametrize("T,E,k,dtype", [
    (256, 8, 2, torch.float32),          # the reference test's and config 1's router
    (1000, 64, 8, torch.float32),        # 8000 slots: four histogram blocks, the last one partial
    (4099, 128, 3, torch.float32),       # k does not divide the block size: tokens straddle histogram blocks
    (32768, 128, 8, torch.bfloat16),     # the expert-parallel configuration's router, 16-bit logits
    (513, 1000, 5, torch.float32),       # widest register tier, ragged last register
    (64, 1024, 32, torch.float16),       # the limits of the fused kernel
    (300, 16, 16, torch.float32),        # k == E
    (1, 8, 2, torch.float32),
    (0, 8, 2, torch.float32),
    (700, 2048, 4, torch.float32),       # beyond the fused kernel: separate kernels, same results
])
def test_route_topk_matches_the_callers_router(T, E, k, dtype, mode, renorm):
    import scattermoe_b200 as sm
    g = torch.Generator().manual_seed(T * 7 + E + k)
    logits = (torch.randn(T, E, generator=g) * 2).to(dtype).cuda()
    gates, ids, (se, ss, off) = sm.route_topk(logits, k, mode, renormalize=renorm)
    assert gates.dtype == torch.float32 and ids.dtype == torch.int64 and gates.shape == ids.shape == (T, k)
    want_g, want_ids = _torch_router(logits, k, mode, renorm)
    if dtype == torch.float32:
        assert torch.equal(ids, want_ids)                 # random fp32 logits: no ties inside a row
    else:
        # 16-bit logits tie often; the stated rule (lower id first) must hold and the selected VALUES must agree
        z = logits.float()
        assert torch.equal(torch.gather(z, 1, ids), torch.gather(z, 1, want_ids))
        same = torch.gather(z, 1, ids)
        tie = same[:, 1:] == same[:, :-1]
        assert bool((ids[:, 1:][tie] > ids[:, :-1][tie]).all())
        want_g = _torch_router(logits, k, mode, renorm)[0]
    torch.testing.assert_close(gates, want_g, rtol=1e-5, atol=1e-6)
    # the routing bookkeeping is exactly the sort of the ids this call returned
    rse, rss, roff = sm.flatten_sort_count(ids, E)
    assert torch.equal(se, rse) and torch.equal(ss, rss) and torch.equal(off, roff)
    sm.check_device_status()


@pytest.mark.parametrize("mode,renorm", [("softmax_topk", True), ("softmax_topk", False), ("topk_softmax", True)])
def test_route_topk_gradient(mode, renorm):
    import scattermoe_b200 as sm
    g = torch.Generator().manual_seed(3)
    T, E, k = 300, 32, 4
    logits = torch.randn(T, E, generator=g).cuda().requires_grad_()
    dg = torch.randn(T, k, generator=g).cuda()
    gates, ids, _ = sm.route_topk(logits, k, mode, renormalize=renorm)
    (got,) = torch.autograd.grad(gates, logits, dg)
    ref_in = logits.detach().clone().requires_grad_()
    want_g, want_ids = _torch_router(ref_in, k, mode, renorm)
    assert torch.equal(ids, want_ids)
    (want,) = torch.autograd.grad(want_g, ref_in, dg)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-6)
