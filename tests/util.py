"""Helpers shared by the tests: golden-vector loading and tolerances."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# tolerances of the parity contract
BF16_RTOL, BF16_ATOL = 2e-2, 2e-2      # bf16 outputs / gradients against the reference
FP32_MAX_ABS = 1e-4                    # fp32 against the dense loop (reference tests/test_mlp.py:83)


def golden_names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        out[k] = a.item() if a.ndim == 0 else torch.from_numpy(a)
    return out


def as_dtype(g, t):
    """Golden float tensors are stored as float32; bring them back to the dtype they were computed in."""
    if t is None:
        return None
    return t.to(torch.bfloat16) if g.get("bf16", False) else t


def assert_close(name, got, want, bf16, atol_scale=1.0):
    """`atol_scale` widens the bf16 absolute tolerance for quantities that are long dot products of
    bf16-rounded terms (the gate gradient sums d_model products of O(1) values rounded to 8 bits)."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, (name, got.shape, want.shape)
    if bf16:
        torch.testing.assert_close(got, want, rtol=BF16_RTOL, atol=BF16_ATOL * atol_scale,
                                   msg=lambda m: "%s: %s" % (name, m))
    else:
        diff = (got - want).abs().max().item() if got.numel() else 0.0
        assert diff < FP32_MAX_ABS, "%s: max abs diff %g" % (name, diff)


def segments_equal_as_sets(sorted_idx_a, sorted_idx_b, offsets):
    """Equality of two slot orders up to the order inside each expert segment."""
    start = 0
    for end in offsets.tolist():
        if not torch.equal(torch.sort(sorted_idx_a[start:end]).values, torch.sort(sorted_idx_b[start:end]).values):
            return False
        start = end
    return True
