"""Expert parallelism for the MoE MLP: experts partitioned across the ranks of one process group, tokens
data-parallel, one exchange step each way.

The reference has no multi-GPU code at all (no torch.distributed import anywhere; README.md:8 leaves
distribution to the surrounding framework), so nothing here mirrors a reference file. The layer computes exactly
what `scattermoe.mlp.GLUMLP` (scattermoe/mlp.py:51-95) computes for the concatenated experts:

    rank r owns experts [r*E/W, (r+1)*E/W) and T/W tokens with their router outputs
    1. plan      stable sort of the local (token, slot) pairs by global expert id = by destination rank;
                 per-(rank, expert) counts exchanged with one small all-to-all; ONE host read of 2W integers
                 (NCCL's all-to-all-v needs its split sizes on the host)
    2. dispatch  rows copied into expert order (`group` kernel), all-to-all-v; received rows land in local HBM
    3. experts   local routing sort (k = 1) -> grouped GEMM -> activation -> grouped GEMM on the received rows
    4. combine   all-to-all-v back, rows return in the sender's expert order, gate-weighted top-k sum
    backward mirrors 4 -> 1; weight gradients stay local (experts are not replicated, no all-reduce).

Row kernels and the sort are injected (`RowOps`) so that the host logic (plans, split sizes, permutations, the
autograd wiring of the collectives) can be exercised by CPU `gloo` ranks in the tests with stand-ins defined by
the tests; the defaults are the CUDA kernels of this package and there is no other implementation in here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from . import activation as _act
from .kernels import ops
from .parallel_experts import flatten_sort_count


class RowOps:
    """The row-level kernels the exchange needs. Default: this package's CUDA kernels."""
    sort = staticmethod(flatten_sort_count)          # (ids (n, k), E) -> (sorted ids, sorted slot idx, inclusive offsets)
    group = staticmethod(ops.group)                  # (A, idx, coeff=None, fan_out=1) -> A[idx // fan_out] * coeff[idx]
    topk_reduce = staticmethod(ops.topk_reduce)      # (expanded (T*k, N), gates or None, T, k) -> (T, N)
    gate_grad = staticmethod(ops.gate_grad)          # (expanded, grad_out, T, k) -> (T, k)


@dataclass
class Plan:
    """Everything both exchange directions need; built once per forward."""
    world: int
    k: int
    tokens: int
    sorted_scattered_idxs: torch.Tensor    # (R_local,) slot of every row in send (expert) order
    inverse: torch.Tensor                  # (R_local,) position in send order of every slot
    send_splits: List[int]                 # rows sent to each rank
    recv_splits: List[int]                 # rows received from each rank
    recv_expert_ids: torch.Tensor          # (R_recv,) LOCAL expert id of every received row
    group: Optional[dist.ProcessGroup]


def split_sizes_from_counts(counts_by_rank_expert: torch.Tensor) -> torch.Tensor:
    """(W, E_local) per-destination per-expert counts -> (W,) rows per destination."""
    return counts_by_rank_expert.sum(dim=1)


def make_plan(expert_idxs: torch.Tensor, num_experts: int, group=None, rowops=RowOps) -> Plan:
    """expert_idxs: (T_local, k) GLOBAL expert ids. Experts are owned in contiguous blocks of E / world."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if num_experts % world:
        raise AssertionError("num_experts (%d) must be divisible by the world size (%d)" % (num_experts, world))
    e_local = num_experts // world
    T, k = expert_idxs.shape
    sorted_e, sorted_idx, offsets = rowops.sort(expert_idxs, num_experts)
    counts = torch.diff(offsets, prepend=offsets.new_zeros(1)).view(world, e_local)      # rows per (dest, expert)
    inverse = torch.empty_like(sorted_idx)
    inverse[sorted_idx] = torch.arange(sorted_idx.numel(), device=sorted_idx.device, dtype=sorted_idx.dtype)
    if world == 1:
        recv_counts = counts
        splits = [int(T * k)]
        return Plan(1, k, T, sorted_idx, inverse, splits, splits, sorted_e.clone(), group)
    recv_counts = torch.empty_like(counts)                                               # rows per (source, expert)
    dist.all_to_all_single(recv_counts, counts.contiguous(), group=group)
    both = torch.stack([split_sizes_from_counts(counts), split_sizes_from_counts(recv_counts)]).cpu()   # the one host read
    send_splits, recv_splits = both[0].tolist(), both[1].tolist()
    local_ids = torch.arange(e_local, device=counts.device, dtype=torch.int64).repeat(world)
    recv_expert_ids = torch.repeat_interleave(local_ids, recv_counts.flatten(), output_size=int(sum(recv_splits)))
    return Plan(world, k, T, sorted_idx, inverse, send_splits, recv_splits, recv_expert_ids, group)


class _AllToAllRows(torch.autograd.Function):
    """all-to-all-v of matrix rows; the gradient travels the opposite way with the split lists swapped."""

    @staticmethod
    def forward(ctx, rows, send_splits, recv_splits, group):
        ctx.cfg = (send_splits, recv_splits, group)
        out = rows.new_empty((int(sum(recv_splits)), rows.size(1)))
        dist.all_to_all_single(out, rows.contiguous(), recv_splits, send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        send_splits, recv_splits, group = ctx.cfg
        back = grad.new_empty((int(sum(send_splits)), grad.size(1)))
        dist.all_to_all_single(back, grad.contiguous(), send_splits, recv_splits, group=group)
        return back, None, None, None


def all_to_all_rows(rows, send_splits, recv_splits, group):
    if len(send_splits) == 1:
        return rows
    return _AllToAllRows.apply(rows, send_splits, recv_splits, group)


class _ToExpertOrder(torch.autograd.Function):
    """x (T, d) -> one row per (token, slot) in send order. Backward: back to slot order, sum over the k slots."""

    @staticmethod
    def forward(ctx, x, plan, rowops):
        ctx.plan, ctx.rowops = plan, rowops
        return rowops.group(x, plan.sorted_scattered_idxs, fan_out=plan.k)

    @staticmethod
    def backward(ctx, grad):
        plan, rowops = ctx.plan, ctx.rowops
        by_slot = rowops.group(grad.contiguous(), plan.inverse, fan_out=1)
        dx = by_slot if plan.k == 1 else rowops.topk_reduce(by_slot, None, plan.tokens, plan.k)
        return dx, None, None


class _GatedCombine(torch.autograd.Function):
    """rows in send order (R, d) + gates (T, k) -> out[t] = sum_j gates[t, j] * row_of_slot(t*k + j)."""

    @staticmethod
    def forward(ctx, rows, gates, plan, rowops):
        by_slot = rowops.group(rows.contiguous(), plan.inverse, fan_out=1)
        ctx.plan, ctx.rowops = plan, rowops
        ctx.save_for_backward(by_slot, gates)
        return rowops.topk_reduce(by_slot, gates, plan.tokens, plan.k)

    @staticmethod
    def backward(ctx, grad):
        plan, rowops = ctx.plan, ctx.rowops
        by_slot, gates = ctx.saved_tensors
        grad = grad.contiguous()
        d_gates = rowops.gate_grad(by_slot, grad, plan.tokens, plan.k).to(gates.dtype) if ctx.needs_input_grad[1] else None
        d_rows = rowops.group(grad, plan.sorted_scattered_idxs, coeff=gates.reshape(-1).to(grad.dtype), fan_out=plan.k)
        return d_rows, d_gates, None, None


def dispatch(x: torch.Tensor, plan: Plan, rowops=RowOps) -> torch.Tensor:
    """(T_local, d) tokens -> (R_recv, d) rows for this rank's experts, ordered by (source rank, local expert)."""
    return all_to_all_rows(_ToExpertOrder.apply(x, plan, rowops), plan.send_splits, plan.recv_splits, plan.group)


def combine(rows: torch.Tensor, gates: torch.Tensor, plan: Plan, rowops=RowOps) -> torch.Tensor:
    """(R_recv, d) expert outputs in received order -> (T_local, d) gate-weighted sums at the owning rank."""
    back = all_to_all_rows(rows, plan.recv_splits, plan.send_splits, plan.group)
    return _GatedCombine.apply(back, gates, plan, rowops)


class ExpertParallelGLUMLP(nn.Module):
    """`GLUMLP` with its experts split across the ranks of `group`. Parameters have the reference's names and
    layouts for the LOCAL experts: experts.weight (E/W, 2*hidden, input), output_experts.weight (E/W, input, hidden);
    concatenating the ranks' tensors along dim 0 gives the reference module's parameters."""

    def __init__(self, input_size, hidden_size, num_experts, top_k, group=None, activation=nn.SiLU()):
        super().__init__()
        from .parallel_experts import ParallelExperts
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if num_experts % world:
            raise AssertionError("num_experts must be divisible by the world size")
        self.num_experts = num_experts
        self.local_experts = num_experts // world
        self.input_size, self.hidden_size = input_size, hidden_size
        self.top_k = min(top_k, num_experts)
        self.group = group
        self.activation = activation
        self.experts = ParallelExperts(self.local_experts, input_size, 2 * hidden_size)
        self.output_experts = ParallelExperts(self.local_experts, hidden_size, input_size)

    def local_expert_mlp(self, rows: torch.Tensor, local_expert_ids: torch.Tensor) -> torch.Tensor:
        """The expert MLP on received rows: every row has exactly one (local) expert, i.e. top_k = 1."""
        routing = flatten_sort_count(local_expert_ids.view(-1, 1), self.local_experts)
        up = self.experts(rows, 1, *routing, grouped_out=True)
        code = _act.resolve_activation(self.activation) if _act.FUSE else None
        if code is None:
            linear_half, gate_half = up.chunk(2, dim=-1)
            hidden = self.activation(gate_half) * linear_half
        else:
            hidden = _act.fused_activation(up, _act.LAYOUT_GLU_SECOND, code)
        return self.output_experts(hidden, 1, *routing, grouped_in=True)

    def forward(self, x: torch.Tensor, expert_p: torch.Tensor, expert_idxs: torch.Tensor):
        lead = x.shape[:-1]
        tokens = x.reshape(-1, x.shape[-1])
        plan = make_plan(expert_idxs.reshape(tokens.size(0), -1), self.num_experts, self.group)
        rows = dispatch(tokens, plan)
        out_rows = self.local_expert_mlp(rows, plan.recv_expert_ids)
        y = combine(out_rows, expert_p.reshape(tokens.size(0), -1), plan)
        return y.view(*lead, y.size(-1))


# ------------------------------------------------------------------------------------------------------------
# NVLink peer-memory exchange: no all-to-all, no regroup copies, no host synchronisation
# ------------------------------------------------------------------------------------------------------------

class PeerBuffers:
    """Symmetric (peer-mapped) buffers of one expert-parallel layer: every rank can address every rank's copy with
    plain loads and stores over NVLink. `shapes`: name -> (shape, dtype). `local[name]` is this rank's tensor,
    `ptrs[name]` the table of all ranks' device pointers the C entry points take. Also holds the flag array of the
    peer-memory barrier."""

    def __init__(self, shapes, device, group=None):
        import ctypes
        import os
        # plain peer mappings only: this code never uses NVLink multicast
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.local, self.ptrs = {}, {}
        for name, (shape, dt) in shapes.items():
            t = symm.empty(shape, dtype=dt, device=device)
            hdl = symm.rendezvous(t, self.group)
            self.local[name] = t
            self.ptrs[name] = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        # flag array of the peer-memory barrier: zeroed here, and no rank may signal before every rank has zeroed
        flags = symm.empty((max(self.world, 8),), dtype=torch.int32, device=device)
        hdl = symm.rendezvous(flags, self.group)
        flags.zero_()
        self.local["flags"] = flags
        self.ptrs["flags"] = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        self.epoch = 0
        self.device = device
        self._token = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.all_reduce(self._token, group=self.group)
        torch.cuda.synchronize(device)

    def barrier(self):
        """Stream-ordered barrier across the ranks on the current stream: kernels enqueued after it on any rank run
        after the kernels (and their peer stores) enqueued before it on every rank. A 32-thread kernel that
        exchanges an epoch number through peer memory; its wait is bounded and reports through the status word.
        (An 8-rank NCCL all-reduce used here first cost ~0.3 ms per barrier, four times per step.)"""
        from . import _lib
        self.epoch += 1
        with torch.cuda.device(self.device):
            _ep_call("smoe_ep_barrier", self.ptrs["flags"], self.rank, self.world, self.epoch,
                     int(BARRIER_LIMIT_CYCLES), _lib.status_word(self.device).data_ptr(), _lib.stream_ptr(self.device))

    def poison_if_a_wait_expired(self, *tensors):
        """After the last barrier of a pass: results computed on the strength of a barrier that gave up waiting become
        NaN (a kernel that reads the status word on the device; no host synchronisation). The status word itself is
        read by `scattermoe_b200.check_device_status()`, which callers should run before `optimizer.step()`."""
        from . import _lib
        with torch.cuda.device(self.device):
            for t in tensors:
                if t is not None and t.numel():
                    _ep_call("smoe_status_poison", _lib.status_word(self.device).data_ptr(), t.data_ptr(),
                             t.numel() * t.element_size(), _lib.stream_ptr(self.device))


class PeerRowBuffers(PeerBuffers):
    """Buffers of the per-slot exchange. At the expert owner: `x` (dispatched tokens), `g` (dispatched output
    gradients), both (capacity, width) and expert-grouped, and `ret` (capacity,) int64 return addresses. At the token
    owner: `yslot`, `dxslot` (tokens*k, width), one row per (token, slot). Capacity is the worst case (all rows of
    all ranks routed to one rank) unless told otherwise, so no routing outcome can overflow a buffer."""

    def __init__(self, capacity_rows: int, slot_rows: int, width: int, dtype, device, group=None):
        self.capacity, self.slot_rows, self.width = int(capacity_rows), int(slot_rows), int(width)
        super().__init__({"x": ((self.capacity, self.width), dtype), "g": ((self.capacity, self.width), dtype),
                          "ret": ((self.capacity,), torch.int64),
                          "yslot": ((self.slot_rows, self.width), dtype), "dxslot": ((self.slot_rows, self.width), dtype)},
                         device, group)


class PeerTokenBuffers(PeerBuffers):
    """Buffers of the exchange that sends every token once per owning rank. At the expert owner: `xtok`, `gtok`
    (token capacity, width) received token / output-gradient rows, `meta` (slot capacity, 2) int64 one record per
    slot in expert-grouped order, `tokmeta` (token capacity, n) int32 one record per received token row. At the token
    owner: `ycomb`, `dxcomb` (tokens * min(k, world), width) one row per (token, owning rank), `dgate` (tokens*k,)
    fp32 gate gradients. Capacities are the worst case (every token of every rank routed here)."""

    def __init__(self, token_capacity: int, local_tokens: int, k: int, width: int, dtype, device, group=None):
        from . import _lib
        world = dist.get_world_size(group if group is not None else dist.group.WORLD)
        self.token_capacity, self.capacity = int(token_capacity), int(token_capacity) * k      # rows: tokens, slots
        self.local_tokens, self.k, self.width = int(local_tokens), int(k), int(width)
        self.slot_rows = self.local_tokens * k
        self.kw = min(k, world)
        self.tm_ints = int(_lib.load().smoe_ep_tokmeta_ints(k))
        if self.tm_ints <= 0:
            raise AssertionError("the once-per-rank exchange lists at most 16 slots per token (k=%d)" % k)
        super().__init__({"xtok": ((self.token_capacity, self.width), dtype), "gtok": ((self.token_capacity, self.width), dtype),
                          "meta": ((self.capacity, 2), torch.int64),
                          "tokmeta": ((self.token_capacity, self.tm_ints), torch.int32),
                          "ycomb": ((self.local_tokens * self.kw, self.width), dtype),
                          "dxcomb": ((self.local_tokens * self.kw, self.width), dtype),
                          "dgate": ((self.slot_rows,), torch.float32)}, device, group)


# Wait limit of the peer-memory barrier in SM clocks (0: the library's default, about one second). A rank that is
# late by more than this (a long host stall between forward and backward, say) makes the others' barrier give up:
# their step then yields NaNs and sets the status word, it does not hang and it does not return plausible numbers.
BARRIER_LIMIT_CYCLES = 0

# Per-slot exchange: the two GEMMs whose results travel home (down-projection in forward, input gradient of the
# up-projection in backward) store them into the home ranks' buffers from their own epilogues. False: separate push
# kernels after the GEMMs (the two forms give bit-identical results).
FUSE_RETURN = True


def _ep_call(name, *args):
    from . import _lib
    rc = getattr(_lib.load(), name)(*args)
    _lib.check(rc, name)


def row_exchange_placement(offsets_all: torch.Tensor, num_experts: int, world: int, rank: int):
    """What `smoe_ep_plan_rows` computes, in tensor operations (the statement the kernel is tested against, and what
    the multi-process CPU tests replay). `offsets_all[s]` = sender s's inclusive per-expert ends. Returns
      dst_off (E,)          first position of this rank's slots of expert e in the owner's expert-grouped buffer
                            (expert-major, then sender)
      local_offsets (E/W,)  inclusive ends of this rank's own experts in its buffer (all senders' slots)"""
    e_local = num_experts // world
    counts_all = torch.diff(offsets_all, dim=1, prepend=offsets_all.new_zeros((world, 1))).clamp_min(0)
    tot = counts_all.sum(0).view(world, e_local)
    ebase = (tot.cumsum(1) - tot).flatten()
    dst_off = (ebase + (counts_all.cumsum(0) - counts_all)[rank]).contiguous()
    local_offsets = tot[rank].cumsum(0).contiguous()
    return dst_off, local_offsets


class _PeerExchangeMLP(torch.autograd.Function):
    """dispatch -> local expert GLU-MLP -> return, forward and backward, on peer row buffers.

    Buffer reuse is safe because of where the four barriers of a step sit: a rank can only start writing a peer's
    buffer for the next phase after every rank has passed the barrier that ends the phase that reads it."""

    @staticmethod
    def forward(ctx, x, gates, expert_idxs, w_up, w_down, layer):
        from . import _lib
        bufs: PeerRowBuffers = layer.buffers
        W, rank, E = bufs.world, bufs.rank, layer.num_experts
        e_local = E // W
        T, k = expert_idxs.shape
        R, d = T * k, x.size(1)
        dev = x.device
        code = _lib.DTYPE_CODE[x.dtype]
        stream = _lib.stream_ptr(dev)
        x = x.contiguous()
        gates = gates.to(x.dtype).contiguous()

        # 1. local routing sort; every rank learns every rank's per-expert offsets (tiny all-gather)
        sorted_e, sorted_idx, offsets = flatten_sort_count(expert_idxs, E)
        offsets_all = torch.empty((W, E), dtype=offsets.dtype, device=dev)
        dist.all_gather_into_tensor(offsets_all, offsets.contiguous(), group=bufs.group)
        # 2. where my rows of expert e start in the owner's buffer; my own experts' inclusive offsets (one small
        # kernel; `row_exchange_placement` below states the arithmetic)
        dst_off = torch.empty(E, dtype=torch.int64, device=dev)
        local_offsets = torch.empty(e_local, dtype=torch.int64, device=dev)
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_plan_rows", offsets_all.data_ptr(), rank, W, E, dst_off.data_ptr(),
                     local_offsets.data_ptr(), stream)
        rows_dev = local_offsets[-1:]
        # 3. dispatch: rows go straight to their final, expert-grouped position on the owning rank
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_dispatch", x.data_ptr(), T, x.stride(0), sorted_e.data_ptr(), sorted_idx.data_ptr(),
                     offsets.data_ptr(), dst_off.data_ptr(), 0, k, bufs.ptrs["x"], bufs.width, bufs.capacity,
                     bufs.ptrs["ret"], rank, R, d, E, W, code, stream)
        bufs.barrier()
        # 4. local experts on the received rows (already grouped: no sort, no copy)
        cap = bufs.capacity
        dummy = layer.dummy_index(cap, dev)
        xb = bufs.local["x"]
        fused = ops.scatter2scatter_act(xb, w_up.permute(0, 2, 1), dummy, dummy, 1, _act.LAYOUT_GLU_SECOND,
                                        layer.act_code, x_grouped=True, expert_offsets=local_offsets)
        if fused is None:       # not a tensor-core case: the grouped GEMM, then the activation kernel
            up = ops.scatter2scatter(xb, w_up.permute(0, 2, 1), dummy, dummy, 1, x_grouped=True, y_grouped=True,
                                     expert_offsets=local_offsets)
            hidden = torch.empty((cap, w_down.size(2)), dtype=x.dtype, device=dev)
            _act._call(False, up, None, hidden, hidden.size(1), _act.LAYOUT_GLU_SECOND, layer.act_code, 1.702, 7.0,
                       rows_dev)
        else:
            up, hidden = fused
        # 5. down-projection; results go home, one row per (token, slot) into the token owner's slot-ordered buffer:
        # stored there by the GEMM's own epilogue as each tile finishes (the rows cross NVLink under the tensor-core
        # work on the next tiles) or, where the tensor-core kernel does not apply, by a push kernel after the GEMM
        if not (FUSE_RETURN and ops.scatter2scatter_to_peers(hidden, w_down.permute(0, 2, 1), local_offsets,
                                                             bufs.local["ret"], bufs.ptrs["yslot"], bufs.width,
                                                             bufs.slot_rows, rank, W)):
            y_rows = ops.scatter2scatter(hidden, w_down.permute(0, 2, 1), dummy, dummy, 1, x_grouped=True,
                                         y_grouped=True, expert_offsets=local_offsets)
            with torch.cuda.device(dev):
                _ep_call("smoe_ep_return", y_rows.data_ptr(), y_rows.stride(0), bufs.local["ret"].data_ptr(),
                         rows_dev.data_ptr(), cap, bufs.ptrs["yslot"], bufs.width, bufs.slot_rows, d, W, rank, e_local,
                         code, stream)
        bufs.barrier()
        out = ops.topk_reduce(bufs.local["yslot"], gates, T, k)
        bufs.poison_if_a_wait_expired(out)
        layer.last_rows_dev = rows_dev          # live rows of the local buffers (device scalar), for accounting
        ctx.layer = layer
        ctx.shape = (T, k, d)
        ctx.save_for_backward(gates, sorted_e, sorted_idx, offsets, dst_off, local_offsets, up, hidden, w_up, w_down)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import _lib
        layer = ctx.layer
        bufs: PeerRowBuffers = layer.buffers
        gates, sorted_e, sorted_idx, offsets, dst_off, local_offsets, up, hidden, w_up, w_down = ctx.saved_tensors
        rows_dev = local_offsets[-1:]
        T, k, d = ctx.shape
        W, E, rank = bufs.world, layer.num_experts, bufs.rank
        dev = grad_out.device
        grad_out = grad_out.to(up.dtype).contiguous()
        code = _lib.DTYPE_CODE[up.dtype]
        stream = _lib.stream_ptr(dev)
        cap = bufs.capacity
        dummy = layer.dummy_index(cap, dev)
        # gate gradient: the per-slot expert outputs are still in the local slot buffer
        d_gates = ops.gate_grad(bufs.local["yslot"], grad_out, T, k) if ctx.needs_input_grad[1] else None
        # gate-scaled output gradient dispatched to the same positions the inputs went to
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_dispatch", grad_out.data_ptr(), T, grad_out.stride(0), sorted_e.data_ptr(),
                     sorted_idx.data_ptr(), offsets.data_ptr(), dst_off.data_ptr(), gates.data_ptr(), k, bufs.ptrs["g"],
                     bufs.width, bufs.capacity, 0, rank, T * k, d, E, W, code, stream)
        bufs.barrier()
        xb, gb = bufs.local["x"], bufs.local["g"]
        e_local = w_up.size(0)
        # input-gradient chain first, its rows start travelling home ...
        # (input gradient of the down-projection and the activation gradient in one launch where the tensor-core
        # kernel applies; only the live rows, which the expert offsets delimit, are read or written)
        d_up = ops.scatter2scatter_act_bwd(gb, w_down, up, local_offsets, _act.LAYOUT_GLU_SECOND, layer.act_code)
        if not (FUSE_RETURN and ops.scatter2scatter_to_peers(d_up, w_up, local_offsets, bufs.local["ret"],
                                                             bufs.ptrs["dxslot"], bufs.width, bufs.slot_rows, rank, W)):
            dx_rows = ops.scatter2scatter(d_up, w_up, dummy, dummy, 1, x_grouped=True, y_grouped=True,
                                          expert_offsets=local_offsets)
            with torch.cuda.device(dev):
                _ep_call("smoe_ep_return", dx_rows.data_ptr(), dx_rows.stride(0), bufs.local["ret"].data_ptr(),
                         rows_dev.data_ptr(), cap, bufs.ptrs["dxslot"], bufs.width, bufs.slot_rows, d, W, rank, e_local,
                         code, stream)
        # ... while the two weight gradients run: the barrier that follows them finds the peers' rows already here
        d_w_down, _ = ops.group_bwd_W(gb, hidden, local_offsets, e_local)
        d_w_up, _ = ops.group_bwd_W(d_up, xb, local_offsets, e_local)
        bufs.barrier()
        dx = ops.topk_reduce(bufs.local["dxslot"], None, T, k) if k > 1 else bufs.local["dxslot"].clone()
        bufs.poison_if_a_wait_expired(dx, d_gates, d_w_up, d_w_down)
        # weight gradients come back as (E, K, N) views of (E, N, K) buffers = the parameters' own layout
        return dx, d_gates, None, d_w_up.permute(0, 2, 1), d_w_down.permute(0, 2, 1), None


@dataclass
class TokenExchangeLocalPlan:
    """What one rank derives from its own routing for the once-per-owning-rank exchange."""
    sorted_e: torch.Tensor        # (R,) global expert of every slot, ascending (stable)
    sorted_idx: torch.Tensor      # (R,) flat slot t*k+j of every sorted position
    offsets: torch.Tensor         # (E,) inclusive per-expert ends of the sorted list
    slot_pos: torch.Tensor        # (R,) sorted position of every slot (inverse of sorted_idx)
    pair_rank: torch.Tensor       # (>= P,) owning rank of every distinct (token, owner) pair, ascending
    pair_slot: torch.Tensor       # (>= P,) the first slot of the pair's token at that owner (token = slot // k)
    pair_offsets: torch.Tensor    # (W,) inclusive per-owner ends of the pair list; P = pair_offsets[-1]
    counts: torch.Tensor          # (E,) slots per expert
    pair_counts: torch.Tensor     # (W,) pairs (= distinct tokens) per owner


def token_exchange_local_plan(ids: torch.Tensor, num_experts: int, world: int, rowops=RowOps) -> TokenExchangeLocalPlan:
    """Slots sorted by expert (as in the per-slot exchange) and the distinct (token, owning rank) pairs sorted by rank:
    a slot opens a pair when no earlier slot of its token has the same owner; the other slots get id -1, which the
    counting sort leaves out (entries of the pair list beyond `pair_offsets[-1]` are not written)."""
    e_local = num_experts // world
    R = ids.numel()
    sorted_e, sorted_idx, offsets = rowops.sort(ids, num_experts)
    slot_pos = torch.empty_like(sorted_idx)
    slot_pos[sorted_idx] = torch.arange(R, device=ids.device, dtype=sorted_idx.dtype)
    owner = ids // e_local
    repeat = (owner.unsqueeze(2) == owner.unsqueeze(1)).tril(-1).any(-1)
    pair_rank, pair_slot, pair_offsets = rowops.sort(torch.where(repeat, -1, owner), world)
    counts = torch.diff(offsets, prepend=offsets.new_zeros(1))
    pair_counts = torch.diff(pair_offsets, prepend=pair_offsets.new_zeros(1))
    return TokenExchangeLocalPlan(sorted_e, sorted_idx, offsets, slot_pos, pair_rank, pair_slot, pair_offsets, counts,
                                  pair_counts)


def token_exchange_placement(gathered: torch.Tensor, num_experts: int, world: int, rank: int):
    """From every rank's counts (`gathered[s] = cat(counts of s, pair_counts of s)`, shape (W, E + W)) to where this
    rank's rows go and what it will hold:
      dst_off (E,)        first position of this rank's slots of expert e in the owner's expert-grouped slot buffer
                          (expert-major, then sender, as in the per-slot exchange)
      local_offsets (E/W,) inclusive ends of this rank's own experts in its slot buffer (all senders' slots)
      tok_base (W,)       first row of this rank's tokens in each owner's token buffer (sender-major)
      src_base (W + 1,)   in this rank's token buffer, the first row of every sender; src_base[-1] = rows held"""
    e_local = num_experts // world
    counts_all, pairs_all = gathered[:, :num_experts], gathered[:, num_experts:]     # [sender, expert], [sender, owner]
    tot = counts_all.sum(0).view(world, e_local)
    ebase = (tot.cumsum(1) - tot).flatten()
    dst_off = (ebase + (counts_all.cumsum(0) - counts_all)[rank]).contiguous()
    local_offsets = tot[rank].cumsum(0).contiguous()
    tok_base = (pairs_all.cumsum(0) - pairs_all)[rank].contiguous()
    src_base = torch.cat([pairs_all.new_zeros(1), pairs_all[:, rank].cumsum(0)]).contiguous()
    return dst_off, local_offsets, tok_base, src_base


class _PeerTokenExchangeMLP(torch.autograd.Function):
    """dispatch -> local expert GLU-MLP -> return on `PeerTokenBuffers`: every token row crosses NVLink once per
    owning rank each way (csrc/ep_dedup.cu). Same results as `_PeerExchangeMLP`; the gate weighting and the gate
    gradient are computed at the expert owner, which receives the gates with the slot records."""

    @staticmethod
    def forward(ctx, x, gates, expert_idxs, w_up, w_down, layer):
        from . import _lib
        bufs: PeerTokenBuffers = layer.buffers
        W, rank, E = bufs.world, bufs.rank, layer.num_experts
        e_local = E // W
        T, k = expert_idxs.shape
        R, d = T * k, x.size(1)
        dev = x.device
        code = _lib.DTYPE_CODE[x.dtype]
        stream = _lib.stream_ptr(dev)
        x = x.contiguous()
        gates = gates.to(x.dtype).contiguous()
        ids = expert_idxs.to(torch.int64).contiguous()

        # 1. plan (device-side integers only; one small all-gather of the counts)
        local = token_exchange_local_plan(ids, E, W)
        gathered = torch.empty((W, E + W), dtype=local.counts.dtype, device=dev)
        dist.all_gather_into_tensor(gathered, torch.cat([local.counts, local.pair_counts]), group=bufs.group)
        placed = token_exchange_placement(gathered, E, W, rank)
        sorted_e, sorted_idx, offsets, slot_pos = local.sorted_e, local.sorted_idx, local.offsets, local.slot_pos
        pair_rank, pair_slot, pair_offsets = local.pair_rank, local.pair_slot, local.pair_offsets
        dst_off, local_offsets, tok_base, src_base = placed
        live_slots, live_tok = local_offsets[-1:], src_base[-1:]
        tok_row = torch.empty((T, W), dtype=torch.int32, device=dev)
        tok_parts = torch.zeros((T,), dtype=torch.int32, device=dev)
        # 2. dispatch: one record per (token, owner) pair, the token rows (once per owner), one record per slot
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_plan_tokens", ids.data_ptr(), gates.data_ptr(), T, k, pair_rank.data_ptr(),
                     pair_slot.data_ptr(), pair_offsets.data_ptr(), tok_base.data_ptr(), slot_pos.data_ptr(),
                     offsets.data_ptr(), dst_off.data_ptr(), tok_row.data_ptr(), tok_parts.data_ptr(), bufs.ptrs["tokmeta"],
                     bufs.token_capacity, bufs.capacity, rank, E, W, code, stream)
            _ep_call("smoe_ep_dispatch", x.data_ptr(), T, x.stride(0), pair_rank.data_ptr(), pair_slot.data_ptr(),
                     pair_offsets.data_ptr(), tok_base.data_ptr(), 0, k, bufs.ptrs["xtok"], bufs.width,
                     bufs.token_capacity, 0, rank, R, d, W, W, code, stream)
            _ep_call("smoe_ep_dispatch_meta", sorted_e.data_ptr(), sorted_idx.data_ptr(), offsets.data_ptr(),
                     dst_off.data_ptr(), gates.data_ptr(), tok_row.data_ptr(), k, bufs.ptrs["meta"], bufs.capacity, rank, R,
                     E, W, code, stream)
        bufs.barrier()
        # 3. owner: token rows into expert order (a copy in local HBM), then the expert MLP as in the per-slot exchange
        cap = bufs.capacity
        dummy = layer.dummy_index(cap, dev)
        xb = torch.empty((cap, d), dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_expand", bufs.local["xtok"].data_ptr(), bufs.width, bufs.token_capacity,
                     bufs.local["meta"].data_ptr(), live_slots.data_ptr(), cap, 0, xb.data_ptr(), xb.stride(0), 0, 0, 0, 0,
                     d, W, code, stream)
        fused = ops.scatter2scatter_act(xb, w_up.permute(0, 2, 1), dummy, dummy, 1, _act.LAYOUT_GLU_SECOND,
                                        layer.act_code, x_grouped=True, expert_offsets=local_offsets)
        if fused is None:
            up = ops.scatter2scatter(xb, w_up.permute(0, 2, 1), dummy, dummy, 1, x_grouped=True, y_grouped=True,
                                     expert_offsets=local_offsets)
            hidden = torch.empty((cap, w_down.size(2)), dtype=x.dtype, device=dev)
            _act._call(False, up, None, hidden, hidden.size(1), _act.LAYOUT_GLU_SECOND, layer.act_code, 1.702, 7.0,
                       live_slots)
        else:
            up, hidden = fused
        y_rows = ops.scatter2scatter(hidden, w_down.permute(0, 2, 1), dummy, dummy, 1, x_grouped=True, y_grouped=True,
                                     expert_offsets=local_offsets)
        # 4. one gate-weighted row per received token goes back to its owner
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_combine", y_rows.data_ptr(), y_rows.stride(0), cap, bufs.local["tokmeta"].data_ptr(),
                     live_tok.data_ptr(), bufs.token_capacity, src_base.data_ptr(), 1, bufs.ptrs["ycomb"], bufs.width,
                     T * bufs.kw, d, k, rank, W, code, stream)
        bufs.barrier()
        out = torch.empty((T, d), dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_sum_parts", bufs.local["ycomb"].data_ptr(), bufs.width, tok_parts.data_ptr(), bufs.kw,
                     out.data_ptr(), out.stride(0), T, d, code, stream)
        bufs.poison_if_a_wait_expired(out)
        layer.last_rows_dev = live_slots
        ctx.layer = layer
        ctx.shape = (T, k, d)
        ctx.gates_dtype = gates.dtype
        ctx.save_for_backward(pair_rank, pair_slot, pair_offsets, tok_base, src_base, local_offsets, tok_parts, xb, up,
                              hidden, y_rows, w_up, w_down)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import _lib
        layer = ctx.layer
        bufs: PeerTokenBuffers = layer.buffers
        (pair_rank, pair_slot, pair_offsets, tok_base, src_base, local_offsets, tok_parts, xb, up, hidden, y_rows, w_up,
         w_down) = ctx.saved_tensors
        live_slots, live_tok = local_offsets[-1:], src_base[-1:]
        T, k, d = ctx.shape
        W, rank = bufs.world, bufs.rank
        dev = grad_out.device
        grad_out = grad_out.to(up.dtype).contiguous()
        code = _lib.DTYPE_CODE[up.dtype]
        stream = _lib.stream_ptr(dev)
        cap = bufs.capacity
        e_local = w_up.size(0)
        # the output gradient of every token goes, un-weighted and once, to each rank that owns one of its slots
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_dispatch", grad_out.data_ptr(), T, grad_out.stride(0), pair_rank.data_ptr(),
                     pair_slot.data_ptr(), pair_offsets.data_ptr(), tok_base.data_ptr(), 0, k, bufs.ptrs["gtok"], bufs.width,
                     bufs.token_capacity, 0, rank, T * k, d, W, W, code, stream)
        bufs.barrier()
        # owner: expand with the gate applied; the same pass computes every slot's gate gradient (its saved expert
        # output times the un-weighted output gradient) and stores it at the token owner
        gb = torch.empty((cap, d), dtype=up.dtype, device=dev)
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_expand", bufs.local["gtok"].data_ptr(), bufs.width, bufs.token_capacity,
                     bufs.local["meta"].data_ptr(), live_slots.data_ptr(), cap, 1, gb.data_ptr(), gb.stride(0),
                     y_rows.data_ptr(), y_rows.stride(0), bufs.ptrs["dgate"], T * k, d, W, code, stream)
        dummy = layer.dummy_index(cap, dev)
        d_up = ops.scatter2scatter_act_bwd(gb, w_down, up, local_offsets, _act.LAYOUT_GLU_SECOND, layer.act_code)
        dx_rows = ops.scatter2scatter(d_up, w_up, dummy, dummy, 1, x_grouped=True, y_grouped=True,
                                      expert_offsets=local_offsets)
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_combine", dx_rows.data_ptr(), dx_rows.stride(0), cap, bufs.local["tokmeta"].data_ptr(),
                     live_tok.data_ptr(), bufs.token_capacity, src_base.data_ptr(), 0, bufs.ptrs["dxcomb"], bufs.width,
                     T * bufs.kw, d, k, rank, W, code, stream)
        # the rows travel home while the two weight gradients run
        d_w_down, _ = ops.group_bwd_W(gb, hidden, local_offsets, e_local)
        d_w_up, _ = ops.group_bwd_W(d_up, xb, local_offsets, e_local)
        bufs.barrier()
        dx = torch.empty((T, d), dtype=up.dtype, device=dev)
        with torch.cuda.device(dev):
            _ep_call("smoe_ep_sum_parts", bufs.local["dxcomb"].data_ptr(), bufs.width, tok_parts.data_ptr(), bufs.kw,
                     dx.data_ptr(), dx.stride(0), T, d, code, stream)
        d_gates = bufs.local["dgate"].view(T, k).to(ctx.gates_dtype) if ctx.needs_input_grad[1] else None
        bufs.poison_if_a_wait_expired(dx, d_gates, d_w_up, d_w_down)
        return dx, d_gates, None, d_w_up.permute(0, 2, 1), d_w_down.permute(0, 2, 1), None


class _PeerChunk:
    """State of one pipeline chunk of a peer-memory layer: its own buffers (so chunks never touch each other's
    rows or flags), its stream, and the bits of layer configuration the autograd function needs."""

    def __init__(self, num_experts, act_code):
        self.num_experts, self.act_code = num_experts, act_code
        self.buffers: Optional[PeerRowBuffers] = None
        self.stream = None
        self.last_rows_dev = None
        self._dummy = None

    def dummy_index(self, n, device):
        """Index tensors are not read when both sides of a grouped GEMM are in expert order; the operator's
        signature still wants them."""
        if self._dummy is None or self._dummy.numel() != n or self._dummy.device != device:
            self._dummy = torch.zeros(n, dtype=torch.int64, device=device)
        return self._dummy


class PeerExpertParallelGLUMLP(ExpertParallelGLUMLP):
    """Same layer and parameters as `ExpertParallelGLUMLP`, with the two all-to-all-v exchanges replaced by
    kernels that write the peers' row buffers directly over NVLink (csrc/ep.cu): the dispatched rows land
    expert-grouped at the owner, results are pushed back to their slots, and nothing is read back to the host.
    16-bit dtypes, input and hidden sizes that are multiples of 8, SiLU / GELU / ReLU gate activations.

    `chunks` > 1 splits the local tokens into that many independent pipelines on their own streams and buffers:
    while one chunk's rows cross NVLink the other chunk's grouped GEMMs run, in forward and (because autograd
    replays every node on the stream of its forward) in backward. Weight gradients of the chunks are summed by
    autograd.

    The buffers belong to the layer and are reused by every step: run one forward (+ backward) at a time per
    layer, with the same number of steps and the same number of local tokens per step on every rank.
    """

    def __init__(self, input_size, hidden_size, num_experts, top_k, group=None, activation=nn.SiLU(),
                 capacity_rows=None, global_tokens=None, chunks=1, once_per_rank=None):
        super().__init__(input_size, hidden_size, num_experts, top_k, group=group, activation=activation)
        # once_per_rank: send every token row once per owning rank (csrc/ep_dedup.cu) instead of once per slot.
        # Default: when that saves at least 70 % of the rows. The per-slot exchange returns its rows from the epilogue
        # of the GEMM that makes them (hidden under the tensor-core work) while this one adds passes over local HBM at
        # the owner: measured on k = 8, E = 128 the two tie when 75 % of the rows are saved (2 ranks) and the per-slot
        # exchange wins at 55 % and 34 % (4 and 8 ranks). With uniform routing a token's top_k slots fall on about
        # world * (1 - (1 - 1/world) ** top_k) distinct ranks.
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        owners = world * (1.0 - (1.0 - 1.0 / world) ** self.top_k)
        if once_per_rank is None:
            once_per_rank = 1 < self.top_k <= 16 and owners <= 0.3 * self.top_k
        self.once_per_rank = bool(once_per_rank)
        if self.once_per_rank and not (1 <= self.top_k <= 16):
            raise AssertionError("once_per_rank needs top_k <= 16")
        self.act_code = _act.resolve_activation(activation)
        if self.act_code is None:
            raise AssertionError("PeerExpertParallelGLUMLP needs an activation this library fuses (SiLU, GELU, ReLU)")
        if input_size % 8 or hidden_size % 8:
            raise AssertionError("input_size and hidden_size must be multiples of 8")
        self._capacity_arg, self._global_tokens = capacity_rows, global_tokens
        self.chunks = max(1, int(chunks))
        self._chunk_state = [_PeerChunk(num_experts, self.act_code) for _ in range(self.chunks)]

    def live_row_fraction(self) -> float:
        """Live rows / capacity of the local receive buffers in the last step (reads device scalars)."""
        live = sum(float(c.last_rows_dev.item()) for c in self._chunk_state if c.last_rows_dev is not None)
        cap = sum(c.buffers.capacity for c in self._chunk_state if c.buffers is not None)
        return live / cap if cap else 1.0

    def _ensure_buffers(self, x, chunk_rows):
        world = dist.get_world_size(self.group)
        for c in self._chunk_state:
            if c.buffers is not None:
                if c.buffers.slot_rows != chunk_rows:
                    raise AssertionError("this layer's peer buffers were sized for %d local (token, slot) rows per "
                                         "chunk, got %d" % (c.buffers.slot_rows, chunk_rows))
                continue
            cap = self._capacity_arg
            if cap is None:
                cap = (self._global_tokens * self.top_k) if self._global_tokens else chunk_rows * self.chunks * world
            cap = ((int(cap) + self.chunks - 1) // self.chunks + 127) // 128 * 128
            if self.once_per_rank:
                k = self.top_k
                c.buffers = PeerTokenBuffers((cap + k - 1) // k, chunk_rows // k, k, self.input_size, x.dtype, x.device,
                                             self.group)
            else:
                c.buffers = PeerRowBuffers(cap, chunk_rows, self.input_size, x.dtype, x.device, self.group)
            c.stream = torch.cuda.Stream(device=x.device) if self.chunks > 1 else None

    def forward(self, x: torch.Tensor, expert_p: torch.Tensor, expert_idxs: torch.Tensor):
        if x.dtype not in (torch.bfloat16, torch.float16):
            raise AssertionError("PeerExpertParallelGLUMLP runs in bfloat16 / float16")
        lead = x.shape[:-1]
        tokens = x.reshape(-1, x.shape[-1])
        T = tokens.size(0)
        idx = expert_idxs.reshape(T, -1)
        gates = expert_p.reshape(T, -1)
        if T % self.chunks:
            raise AssertionError("the number of local tokens (%d) must be divisible by chunks=%d" % (T, self.chunks))
        tc = T // self.chunks
        self._ensure_buffers(tokens, tc * idx.size(1))
        w_up, w_down = self.experts.weight, self.output_experts.weight
        exchange = _PeerTokenExchangeMLP if self.once_per_rank else _PeerExchangeMLP
        if self.chunks == 1:
            y = exchange.apply(tokens, gates, idx, w_up, w_down, self._chunk_state[0])
            return y.view(*lead, y.size(-1))
        cur = torch.cuda.current_stream(tokens.device)
        outs = []
        for i, c in enumerate(self._chunk_state):
            c.stream.wait_stream(cur)
            sl = slice(i * tc, (i + 1) * tc)
            with torch.cuda.stream(c.stream):
                outs.append(exchange.apply(tokens[sl], gates[sl], idx[sl], w_up, w_down, c))
        for c, o in zip(self._chunk_state, outs):
            cur.wait_stream(c.stream)
            o.record_stream(cur)
        y = torch.cat(outs, dim=0)
        return y.view(*lead, y.size(-1))
