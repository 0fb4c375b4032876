"""Expert-parallel layer on GPUs: with one rank it must equal `GLUMLP`; with two ranks (NCCL, when the box has two
GPUs) each rank's outputs and gradients must equal the matching slices of the single-GPU layer on the gathered
problem. Ranks leave only after all work is done; NVLS is switched off for the child processes."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _problem(T=512, d=256, F=128, E=8, k=2, seed=5):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    x = torch.randn(T, d, generator=g).to(bf)
    p, idx = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), k)
    w1 = (torch.randn(E, 2 * F, d, generator=g) * 0.05).to(bf)
    w2 = (torch.randn(E, d, F, generator=g) * 0.05).to(bf)
    dy = torch.randn(T, d, generator=g).to(bf)
    return x, p.to(bf), idx, w1, w2, dy


def _reference_on(device, x, p, idx, w1, w2, dy):
    import scattermoe_b200 as sm
    E, F2, d = w1.shape
    m = sm.mlp.GLUMLP(d, F2 // 2, E, idx.size(1)).to(device).bfloat16()
    with torch.no_grad():
        m.experts.weight.copy_(w1)
        m.output_experts.weight.copy_(w2)
    xx, pp = x.to(device).requires_grad_(), p.to(device).requires_grad_()
    y = m(xx, pp, idx.to(device))
    g = torch.autograd.grad(y, [xx, pp, m.experts.weight, m.output_experts.weight], dy.to(device))
    return [t.float().cpu() for t in [y] + list(g)]


def _close(name, got, want):
    s = max(1.0, want.abs().max().item() / 4)
    torch.testing.assert_close(got.float().cpu() / s, want / s, rtol=2e-2, atol=2e-2, msg=lambda m: name + ": " + m)


def test_single_rank_equals_glumlp():
    import scattermoe_b200 as sm
    from scattermoe_b200.expert_parallel import ExpertParallelGLUMLP
    dev = torch.device("cuda", 0)
    x, p, idx, w1, w2, dy = _problem()
    want = _reference_on(dev, x, p, idx, w1, w2, dy)
    m = ExpertParallelGLUMLP(x.size(1), w2.size(2), w1.size(0), idx.size(1)).to(dev).bfloat16()
    with torch.no_grad():
        m.experts.weight.copy_(w1)
        m.output_experts.weight.copy_(w2)
    xx, pp = x.to(dev).requires_grad_(), p.to(dev).requires_grad_()
    y = m(xx, pp, idx.to(dev))
    g = torch.autograd.grad(y, [xx, pp, m.experts.weight, m.output_experts.weight], dy.to(dev))
    for name, got, ref in zip(("y", "dx", "dp", "dw1", "dw2"), [y] + list(g), want):
        _close(name, got, ref)
    sm.check_device_status(dev)


def _worker(rank, world, port, ret, peer=False, chunks=1, problem=None, once_per_rank=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import scattermoe_b200 as sm
        from scattermoe_b200.expert_parallel import ExpertParallelGLUMLP, PeerExpertParallelGLUMLP
        x, p, idx, w1, w2, dy = _problem(**(problem or {}))
        T, E = x.size(0), w1.size(0)
        tl, el = T // world, E // world
        ts, es = slice(rank * tl, (rank + 1) * tl), slice(rank * el, (rank + 1) * el)
        want = _reference_on(dev, x, p, idx, w1, w2, dy)
        if peer:
            m = PeerExpertParallelGLUMLP(x.size(1), w2.size(2), E, idx.size(1), chunks=chunks,
                                         once_per_rank=once_per_rank).to(dev).bfloat16()
        else:
            m = ExpertParallelGLUMLP(x.size(1), w2.size(2), E, idx.size(1)).to(dev).bfloat16()
        with torch.no_grad():
            m.experts.weight.copy_(w1[es])
            m.output_experts.weight.copy_(w2[es])
        xx, pp = x[ts].to(dev).requires_grad_(), p[ts].to(dev).requires_grad_()
        for _ in range(3):      # repeated: later passes run on warm communicators and reused buffers
            y = m(xx, pp, idx[ts].to(dev))
            g = torch.autograd.grad(y, [xx, pp, m.experts.weight, m.output_experts.weight], dy[ts].to(dev))
        _close("y", y, want[0][ts]); _close("dx", g[0], want[1][ts]); _close("dp", g[1], want[2][ts])
        _close("dw1", g[2], want[3][es]); _close("dw2", g[3], want[4][es])
        sm.check_device_status(dev)
        torch.cuda.synchronize()
        dist.barrier()
        ret[rank] = "ok"
    except Exception:
        import traceback
        ret[rank] = "FAILED: " + traceback.format_exc()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("problem", [None, dict(T=1024, d=256, F=128, E=16, k=8, seed=9)], ids=["k2_E8", "k8_E16"])
@pytest.mark.parametrize("peer,chunks,once", [(False, 1, None), (True, 1, False), (True, 1, True), (True, 2, False), (True, 2, True)],
                         ids=["nccl_all_to_all", "nvlink_per_slot", "nvlink_once_per_rank", "nvlink_per_slot_2_chunks",
                              "nvlink_once_per_rank_2_chunks"])
def test_two_ranks_equal_the_single_gpu_layer(peer, chunks, once, problem):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret, peer, chunks, problem, once)) for r in range(2)]
        for q in procs:
            q.start()
        for q in procs:
            q.join(timeout=240)
        for q in procs:
            if q.is_alive():
                q.terminate()
                raise AssertionError("a rank did not finish")
        assert {r: ret.get(r) for r in range(2)} == {0: "ok", 1: "ok"}


def test_barrier_that_nobody_answers_gives_up_and_is_loud():
    """A bounded wait that runs out (a flag that nothing sets; no fault, no hang): the kernel returns, the status
    word says which peer stayed silent, `check_device_status` raises, and `smoe_status_poison` turns results that
    were computed on the strength of that barrier into NaNs. One GPU plays rank 0 of a world of 2 whose rank 1 never
    signals (both entries of the flag table point at the same local array; slot 1 of it is never written)."""
    import ctypes
    import scattermoe_b200 as sm
    from scattermoe_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    sm.check_device_status(dev)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    table = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    status = _lib.status_word(dev)
    results = torch.ones(1000, dtype=torch.bfloat16, device=dev)[3:]          # deliberately not 16-byte aligned
    untouched = torch.ones(64, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        # nothing expired yet: the poison kernel must leave the buffer alone
        assert lib.smoe_status_poison(status.data_ptr(), untouched.data_ptr(), untouched.numel() * 4,
                                      _lib.stream_ptr(dev)) == 0
        rc = lib.smoe_ep_barrier(table, 0, 2, 1, 5_000_000, status.data_ptr(), _lib.stream_ptr(dev))   # ~3 ms of clocks
        assert rc == 0, _lib.last_error()
        assert lib.smoe_status_poison(status.data_ptr(), results.data_ptr(), results.numel() * 2,
                                      _lib.stream_ptr(dev)) == 0
    torch.cuda.synchronize()                      # the kernel returned
    assert status.tolist() == [2, 100, 1, 1]
    assert bool((untouched == 1).all())
    assert bool(torch.isnan(results.float()).all())
    with pytest.raises(RuntimeError, match="gave up waiting"):
        sm.check_device_status(dev)
    sm.check_device_status(dev)                   # the word was cleared by the check
    # a barrier every party answers passes: world of 1
    one = (ctypes.c_void_p * 1)(flags.data_ptr())
    with torch.cuda.device(dev):
        assert lib.smoe_ep_barrier(one, 0, 1, 2, 0, status.data_ptr(), _lib.stream_ptr(dev)) == 0
    sm.check_device_status(dev)


@pytest.mark.parametrize("store_bytes", [64, 128, 256])
@pytest.mark.parametrize("rank", [0, 2])
@pytest.mark.parametrize("K,N", [(128, 256), (256, 512), (64, 136)])
def test_gemm_that_returns_its_rows_equals_gemm_then_push(rank, K, N, store_bytes, monkeypatch):
    """`smoe_scatter2scatter_to_peers` against `smoe_scatter2scatter` + `smoe_ep_return` on the same inputs, bit for
    bit. One GPU plays the owner; the four "ranks" its rows return to are four buffers of this GPU (a peer pointer is
    just an address). Ragged local experts (one empty, one larger than a tile), a buffer larger than its live rows,
    and two malformed return addresses, whose rows must be dropped by both forms. All three store widths of the
    epilogue."""
    import ctypes
    from scattermoe_b200 import _lib
    from scattermoe_b200.kernels import ops
    # contiguous bytes of a row per store instruction of the epilogue (the library reads this at every launch)
    monkeypatch.setenv("SMOE_PEER_STORE_BYTES", str(store_bytes))
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(100 + K + rank)
    world, slot_rows, cap = 4, 700, 1024
    counts = torch.tensor([130, 0, 301, 57, 200])
    live, E = int(counts.sum()), counts.numel()
    offsets = counts.cumsum(0).to(dev)
    X = torch.randn(cap, K, generator=g).to(torch.bfloat16).to(dev)
    W = (torch.randn(E, K, N, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    # every live row has its own (rank, slot) home
    homes = torch.randperm(world * slot_rows, generator=g)[:live]
    ret = torch.full((cap,), -1, dtype=torch.int64)
    ret[:live] = ((homes // slot_rows) << 40) | (homes % slot_rows)
    ret[5] = (7 << 40) | 3                      # rank outside the world
    ret[140] = (1 << 40) | (slot_rows + 9)      # row outside the peer buffer
    ret = ret.to(dev)
    dummy = torch.zeros(cap, dtype=torch.int64, device=dev)

    def buffers():
        b = [torch.full((slot_rows, N), -7.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        return b, (ctypes.c_void_p * world)(*[t.data_ptr() for t in b])

    two, two_ptrs = buffers()
    y = ops.scatter2scatter(X, W, dummy, dummy, 1, x_grouped=True, y_grouped=True, expert_offsets=offsets)
    rows_dev = offsets[-1:].contiguous()
    with torch.cuda.device(dev):
        rc = _lib.load().smoe_ep_return(y.data_ptr(), y.stride(0), ret.data_ptr(), rows_dev.data_ptr(), cap, two_ptrs, N,
                                        slot_rows, N, world, rank, E, _lib.DTYPE_CODE[torch.bfloat16], _lib.stream_ptr(dev))
    assert rc == 0, _lib.last_error()
    one, one_ptrs = buffers()
    fits = K % 8 == 0 and N % 8 == 0
    assert ops.scatter2scatter_to_peers(X, W, offsets, ret, one_ptrs, N, slot_rows, rank, world) == fits
    torch.cuda.synchronize()
    import scattermoe_b200 as sm
    sm.check_device_status(dev)
    written = 0
    for a, b in zip(one, two):
        assert torch.equal(a, b)
        written += int((b != -7.0).any(1).sum())
    assert written == live - 2


@pytest.mark.parametrize("world,E", [(1, 8), (2, 8), (8, 128), (4, 1024)])
def test_row_placement_kernel_equals_its_statement(world, E):
    """`smoe_ep_plan_rows` against `row_exchange_placement` (tensor operations), bit for bit, for every rank."""
    from scattermoe_b200 import _lib
    from scattermoe_b200 import expert_parallel as ep
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(E + world)
    counts = torch.randint(0, 50, (world, E), generator=g)
    counts[0, : E // 2] = 0                                           # experts nobody on rank 0 routes to
    offsets_all = counts.cumsum(1).to(dev)
    for rank in range(world):
        want_dst, want_loc = ep.row_exchange_placement(offsets_all, E, world, rank)
        dst = torch.full((E,), -1, dtype=torch.int64, device=dev)
        loc = torch.full((E // world,), -1, dtype=torch.int64, device=dev)
        with torch.cuda.device(dev):
            rc = _lib.load().smoe_ep_plan_rows(offsets_all.data_ptr(), rank, world, E, dst.data_ptr(), loc.data_ptr(),
                                               _lib.stream_ptr(dev))
        assert rc == 0, _lib.last_error()
        assert torch.equal(dst, want_dst) and torch.equal(loc, want_loc)
