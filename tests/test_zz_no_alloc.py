"""The allocation-free routing entry point (`smoe_sort_count_static`), called through the C ABI.

Some hosts of this library cannot allocate device memory when they call it (an inference server that gave all of
HBM to its own arena at start-up, an embedder with no device allocator): for them the sort keeps its block
histograms in an array built into the library. The test drives both entry points with the same device buffers,
twice in a row with different inputs, and requires bit-identical outputs; the second call also proves that
whatever the first call left in the shared array does no harm. Collected last so that a run that stops at the
first failure has already run every other test; passes on its own in a fresh process as well.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_static, ids, E):
    from scattermoe_b200 import _lib
    R = ids.numel()
    dev = ids.device
    out = [torch.full((R,), -1, dtype=torch.int64, device=dev), torch.full((R,), -1, dtype=torch.int64, device=dev),
           torch.full((E,), -1, dtype=torch.int64, device=dev)]
    stream = _lib.stream_ptr(dev)
    if fn_static:
        rc = lib.smoe_sort_count_static(ids.data_ptr(), R, E, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                        stream)
    else:
        nbytes = lib.smoe_sort_count_workspace_bytes(R, E)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        rc = lib.smoe_sort_count(ids.data_ptr(), R, E, out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(),
                                 ws.data_ptr(), nbytes, stream)
    return rc, out


def test_static_scratch_sort_matches_workspace_sort_twice_in_a_row():
    from scattermoe_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(11)
    # call 1: a large, many-expert problem that fills much of the scratch; call 2: a small one right after it
    for R, E in [(262144, 64), (5000, 8), (2048 * 9 + 17, 128)]:
        ids = torch.randint(0, E, (R,), generator=g, dtype=torch.int64)
        ids[ids == 1] = 0                                   # an empty expert
        ids = ids.to(dev)
        rc_a, a = _call(lib, True, ids, E)
        rc_b, b = _call(lib, False, ids, E)
        torch.cuda.synchronize()
        assert rc_a == 0, _lib.last_error()
        assert rc_b == 0, _lib.last_error()
        for x, y in zip(a, b):
            assert torch.equal(x, y)
        assert int(a[2][-1]) == R and bool((a[0][1:] >= a[0][:-1]).all())


@pytest.mark.parametrize("R,E", [(1 << 21, 128), (2048 * 32, 4096), (2048 * 1024 - 5, 128)])
def test_static_scratch_accepts_requests_at_its_capacity(R, E):
    """ceil(R / 2048) * E equal to the capacity (the header's own example, 2^21 slots at 128 experts, and the widest
    expert range) must be served, with the same bits as the workspace entry point."""
    from scattermoe_b200 import _lib
    lib = _lib.load()
    assert -(-R // 2048) * E == lib.smoe_sort_count_static_capacity()
    dev = torch.device("cuda", 0)
    ids = torch.randint(0, E, (R,), generator=torch.Generator().manual_seed(R % 1000 + E), dtype=torch.int64).to(dev)
    rc_a, a = _call(lib, True, ids, E)
    rc_b, b = _call(lib, False, ids, E)
    torch.cuda.synchronize()
    assert rc_a == 0, _lib.last_error()
    assert rc_b == 0, _lib.last_error()
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    assert int(a[2][-1]) == R


def test_static_scratch_rejects_oversized_requests_without_touching_memory():
    from scattermoe_b200 import _lib
    lib = _lib.load()
    cap = lib.smoe_sort_count_static_capacity()
    assert cap == 128 * 1024
    E = 4096
    R = 2048 * (cap // E) + 1                               # one block of ids too many
    rc = lib.smoe_sort_count_static(256, R, E, 256, 256, 256, None)      # pointers are never dereferenced
    assert rc == 4 and "exceeds the built-in scratch" in _lib.last_error()
    with pytest.raises(RuntimeError):
        _lib.check(rc, "smoe_sort_count_static")
