"""Expert-parallel host logic on CPU ranks (gloo, world size 2 and 4): plans, split sizes, permutations, the autograd
wiring of the two all-to-all-v exchanges. The CUDA row kernels are replaced by torch stand-ins defined HERE (the
product has no CPU implementation); the expert arithmetic is the oracle's dense loop. The result of the sharded
run must equal the single-process oracle on the gathered problem, forward and every gradient."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))


class TorchRowOps:
    """CPU stand-ins with the signatures of scattermoe_b200.expert_parallel.RowOps."""

    @staticmethod
    def sort(ids, E):
        import scattermoe_oracle as oracle
        return oracle.flatten_sort_count(ids, E)

    @staticmethod
    def group(A, idx, coeff=None, fan_out=1):
        rows = A[torch.div(idx, fan_out, rounding_mode="floor")]
        return rows if coeff is None else rows * coeff.reshape(-1)[idx][:, None]

    @staticmethod
    def topk_reduce(expanded, gates, T, k):
        v = expanded.view(T, k, -1)
        return v.sum(1) if gates is None else (gates.unsqueeze(1) @ v).squeeze(1)

    @staticmethod
    def gate_grad(expanded, grad_out, T, k):
        return (expanded.view(T, k, -1) @ grad_out.unsqueeze(-1)).squeeze(-1)


def _problem(seed=0, T=48, d=16, F=12, E=8, k=3):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, d, generator=g, dtype=torch.float64)
    logits = torch.randn(T, E, generator=g, dtype=torch.float64)
    logits[:, 2] -= 50.0                      # an expert nobody routes to
    p, idx = torch.topk(torch.softmax(logits, -1), k)
    w1 = torch.randn(E, d, 2 * F, generator=g, dtype=torch.float64) * 0.3
    w2 = torch.randn(E, F, d, generator=g, dtype=torch.float64) * 0.3
    dy = torch.randn(T, d, generator=g, dtype=torch.float64)
    return x, p, idx, w1, w2, dy


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import scattermoe_oracle as oracle
        from scattermoe_b200 import expert_parallel as ep
        x, p, idx, w1, w2, dy = _problem()
        T, E = x.size(0), w1.size(0)
        tl, el = T // world, E // world
        sl = slice(rank * tl, (rank + 1) * tl)
        xl = x[sl].clone().requires_grad_()
        pl = p[sl].clone().requires_grad_()
        w1l = w1[rank * el:(rank + 1) * el].clone().requires_grad_()
        w2l = w2[rank * el:(rank + 1) * el].clone().requires_grad_()

        plan = ep.make_plan(idx[sl], E, rowops=TorchRowOps)
        assert sum(plan.send_splits) == tl * idx.size(1)
        assert plan.recv_expert_ids.numel() == sum(plan.recv_splits)
        rows = ep.dispatch(xl, plan, rowops=TorchRowOps)
        # dense expert arithmetic on the received rows (each row has one local expert)
        out = torch.zeros(rows.size(0), x.size(1), dtype=rows.dtype)
        for e in range(el):
            sel = (plan.recv_expert_ids == e).nonzero().squeeze(-1)
            if sel.numel():
                h = oracle.act_glu_second_half(rows[sel] @ w1l[e])
                out = out.index_add(0, sel, h @ w2l[e])
        y = ep.combine(out, pl, plan, rowops=TorchRowOps)
        grads = torch.autograd.grad(y, [xl, pl, w1l, w2l], dy[sl])

        want = oracle.moe_mlp_forward_backward(x, p, idx, w1, w2, None, None, oracle.act_glu_second_half, dy,
                                               compute_dtype=torch.float64)
        checks = [("y", y, want["y"][sl]), ("dx", grads[0], want["d_x"][sl]), ("dp", grads[1], want["d_expert_p"][sl]),
                  ("dw1", grads[2], want["d_w1"][rank * el:(rank + 1) * el]),
                  ("dw2", grads[3], want["d_w2"][rank * el:(rank + 1) * el])]
        for name, got, ref in checks:
            err = (got.detach() - ref).abs().max().item()
            assert err < 1e-9, "%s rank %d: %g" % (name, rank, err)
        # the counts every rank received must add up to the global histogram of its experts
        hist = torch.bincount(idx.flatten(), minlength=E)[rank * el:(rank + 1) * el]
        assert torch.equal(torch.bincount(plan.recv_expert_ids, minlength=el), hist)
        ret[rank] = "ok"
    except Exception as e:  # surface the failure in the parent
        import traceback
        ret[rank] = "FAILED: " + traceback.format_exc()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_exchange_on_gloo_ranks(world):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=180)
        for p in procs:
            if p.is_alive():
                p.terminate()
                raise AssertionError("a rank did not finish")
        assert {r: ret.get(r) for r in range(world)} == {r: "ok" for r in range(world)}


def test_plan_on_a_single_process_is_the_plain_routing_sort():
    """Without a process group the plan degenerates to one rank that keeps every row."""
    from scattermoe_b200 import expert_parallel as ep
    x, p, idx, w1, w2, dy = _problem(seed=3)
    plan = ep.make_plan(idx, w1.size(0), rowops=TorchRowOps)
    assert plan.world == 1 and plan.send_splits == plan.recv_splits == [idx.numel()]
    assert torch.equal(plan.inverse[plan.sorted_scattered_idxs], torch.arange(idx.numel()))
    assert torch.equal(plan.recv_expert_ids, torch.sort(idx.flatten()).values)
    rows = ep.dispatch(x, plan, rowops=TorchRowOps)
    assert torch.equal(rows, x[plan.sorted_scattered_idxs // idx.size(1)])


@pytest.mark.parametrize("world,E,k", [(1, 8, 2), (2, 8, 2), (4, 16, 8), (8, 128, 8)])
def test_per_slot_exchange_placement_fills_every_owner_buffer_exactly(world, E, k):
    """`row_exchange_placement` (the arithmetic `smoe_ep_plan_rows` runs on the device) for every rank of a world,
    with the dispatch stores played on the host: every owner's buffer must end up holding each of its slots exactly
    once, grouped by local expert and, inside an expert, ordered by sending rank; `local_offsets` must delimit the
    experts."""
    from scattermoe_b200 import expert_parallel as ep
    g = torch.Generator().manual_seed(world * 100 + E)
    T, e_local = 96, E // world
    ids = [torch.topk(torch.rand(T, E, generator=g), k).indices for _ in range(world)]
    if world > 1:
        ids[1] = ids[1] % e_local                                  # one sender routes everything to rank 0
    sorts = [TorchRowOps.sort(i, E) for i in ids]                  # (sorted ids, sorted slots, inclusive offsets)
    offsets_all = torch.stack([s[2] for s in sorts])
    received = [[] for _ in range(world)]                          # per owner: (position, expert, sender)
    placements = [ep.row_exchange_placement(offsets_all, E, world, r) for r in range(world)]
    for sender, (sorted_e, _, offsets) in enumerate(sorts):
        dst_off = placements[sender][0]
        starts = offsets - torch.diff(offsets, prepend=offsets.new_zeros(1))
        for m, e in enumerate(sorted_e.tolist()):
            received[e // e_local].append((int(dst_off[e]) + m - int(starts[e]), e, sender))
    for owner in range(world):
        rows = sorted(received[owner])
        assert [r[0] for r in rows] == list(range(len(rows)))      # a permutation of 0..n-1: no gap, no collision
        assert [(r[1], r[2]) for r in rows] == sorted((r[1], r[2]) for r in rows)      # (expert, sender) order
        local_offsets = placements[owner][1]
        per_expert = [sum(1 for r in rows if r[1] == owner * e_local + j) for j in range(e_local)]
        assert local_offsets.tolist() == torch.tensor(per_expert).cumsum(0).tolist()


# ---- the once-per-owning-rank exchange: its plan and placement arithmetic, with the peer stores played on the host ----

class SkippingSort:
    """`RowOps.sort` stand-in that, like the CUDA counting sort, leaves out ids outside [0, E): their entries of the
    two sorted outputs are never written (filled with a poison value here)."""

    @staticmethod
    def sort(ids, E):
        flat = ids.reshape(-1).to(torch.int64)
        valid = (flat >= 0) & (flat < E)
        order = torch.sort(torch.where(valid, flat, torch.full_like(flat, E)), stable=True).indices
        n = int(valid.sum())
        sorted_e = torch.full_like(flat, -7)
        sorted_idx = torch.full_like(flat, -7)
        sorted_e[:n], sorted_idx[:n] = flat[order[:n]], order[:n]
        return sorted_e, sorted_idx, torch.bincount(flat[valid], minlength=E).cumsum(-1)


def _token_exchange_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import scattermoe_oracle as oracle
        from scattermoe_b200 import expert_parallel as ep
        x, p, idx, w1, w2, dy = _problem(seed=11, T=64, E=8, k=4)
        T, E, k, d = x.size(0), w1.size(0), idx.size(1), x.size(1)
        tl, el = T // world, E // world
        sl = slice(rank * tl, (rank + 1) * tl)
        ids, gates, xl = idx[sl], p[sl], x[sl]
        kw = min(k, world)

        local = ep.token_exchange_local_plan(ids, E, world, rowops=SkippingSort)
        mine = torch.cat([local.counts, local.pair_counts])
        everyone = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        gathered = torch.stack(everyone)
        dst_off, local_offsets, tok_base, src_base = ep.token_exchange_placement(gathered, E, world, rank)
        pairs = int(local.pair_offsets[-1])
        # every (token, owner) pair exactly once, owners ascending, tokens ascending inside an owner
        owner_of = ids // el
        want_pairs = sorted({(int(owner_of[t, j]), t) for t in range(tl) for j in range(k)})
        got_pairs = [(int(local.pair_rank[i]), int(local.pair_slot[i]) // k) for i in range(pairs)]
        assert got_pairs == want_pairs

        # what the kernels do, on the host: peer stores become lists of (destination, buffer, row, payload)
        writes = []
        tok_row = {}
        for i in range(pairs):
            w, t = got_pairs[i]
            start = int(local.pair_offsets[w - 1]) if w else 0
            row = int(tok_base[w]) + (i - start)
            tok_row[(t, w)] = row
            owners = sorted({int(o) for o in owner_of[t]})
            slots = [j for j in range(k) if int(owner_of[t, j]) == w]
            pos = []
            for j in slots:
                e = int(ids[t, j])
                seg = int(local.offsets[e - 1]) if e else 0
                pos.append(int(dst_off[e]) + int(local.slot_pos[t * k + j]) - seg)
            writes.append((w, "xtok", row, xl[t]))
            writes.append((w, "tokmeta", row, (rank, t * kw + owners.index(w), pos, [gates[t, j] for j in slots])))
        for m in range(tl * k):
            e, slot = int(local.sorted_e[m]), int(local.sorted_idx[m])
            w, t = e // el, slot // k
            seg = int(local.offsets[e - 1]) if e else 0
            writes.append((w, "meta", int(dst_off[e]) + m - seg, tok_row[(t, w)]))
        inbox = [None] * world
        dist.all_gather_object(inbox, writes)
        bufs = {"xtok": {}, "tokmeta": {}, "meta": {}}
        for sender in inbox:
            for dest, name, row, payload in sender:
                if dest == rank:
                    assert row not in bufs[name], "two stores to row %d of %s" % (row, name)
                    bufs[name][row] = payload
        live_slots, live_tok = int(local_offsets[-1]), int(src_base[-1])
        assert sorted(bufs["meta"]) == list(range(live_slots)) and sorted(bufs["xtok"]) == list(range(live_tok))
        assert sorted(bufs["tokmeta"]) == list(range(live_tok))
        # owner: expand, expert MLP per local expert, gate-weighted sum per received token row, one row back
        xb = torch.stack([bufs["xtok"][bufs["meta"][q]] for q in range(live_slots)]) if live_slots else x.new_zeros((0, d))
        y_rows = torch.zeros_like(xb)
        start = 0
        for e_l, end in enumerate(local_offsets.tolist()):
            e = rank * el + e_l
            if end > start:
                y_rows[start:end] = oracle.act_glu_second_half(xb[start:end] @ w1[e]) @ w2[e]
            start = end
        back = []
        for u in range(live_tok):
            src, ret_row, pos, gs = bufs["tokmeta"][u]
            back.append((src, ret_row, sum(g * y_rows[q] for q, g in zip(pos, gs))))
        inbox = [None] * world
        dist.all_gather_object(inbox, back)
        parts = {}
        for sender in inbox:
            for dest, ret_row, row in sender:
                if dest == rank:
                    assert ret_row not in parts
                    parts[ret_row] = row
        y = torch.stack([sum(parts[t * kw + c] for c in range(len({int(o) for o in owner_of[t]}))) for t in range(tl)])
        want = oracle.dense_moe_mlp(x, p, idx, w1, w2, None, None, oracle.act_glu_second_half, torch.float64)
        err = (y - want[sl]).abs().max().item()
        assert err < 1e-9, "y rank %d: %g" % (rank, err)
        assert len(parts) == sum(len({int(o) for o in owner_of[t]}) for t in range(tl))
        ret[rank] = "ok"
    except Exception:
        import traceback
        ret[rank] = "FAILED: " + traceback.format_exc()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_once_per_owning_rank_exchange_plan_on_gloo_ranks(world):
    """Plan and placement arithmetic of the once-per-owning-rank exchange (token_exchange_local_plan /
    token_exchange_placement): with the peer stores of the CUDA kernels replayed on the host, every buffer row is
    written exactly once, the buffers are dense, and the forward result equals the oracle's dense loop."""
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_token_exchange_worker, args=(r, world, port, ret)) for r in range(world)]
        for q in procs:
            q.start()
        for q in procs:
            q.join(timeout=180)
        for q in procs:
            if q.is_alive():
                q.terminate()
                raise AssertionError("a rank did not finish")
        assert {r: ret.get(r) for r in range(world)} == {r: "ok" for r in range(world)}


@pytest.mark.parametrize("world,k,expect", [(2, 8, True), (4, 8, False), (8, 8, False), (2, 2, False), (8, 2, False),
                                            (1, 8, True), (2, 1, False)])
def test_default_exchange_of_the_peer_layer(world, k, expect, monkeypatch):
    """Which NVLink exchange the layer picks by itself: once per owning rank only where it saves at least 70 % of the
    rows (expected distinct owners of a token's k slots <= 0.3 k), else per slot with the return fused into the GEMM;
    an explicit argument always wins."""
    from scattermoe_b200 import expert_parallel as ep
    monkeypatch.setattr(ep.dist, "is_initialized", lambda: True)
    monkeypatch.setattr(ep.dist, "get_world_size", lambda group=None: world)
    monkeypatch.setattr(ep.dist, "get_rank", lambda group=None: 0)
    E = 16 * world
    layer = ep.PeerExpertParallelGLUMLP(64, 32, E, k)
    assert layer.once_per_rank is expect
    assert ep.PeerExpertParallelGLUMLP(64, 32, E, k, once_per_rank=not expect).once_per_rank is (not expect and k > 0)
    assert ep.FUSE_RETURN is True
