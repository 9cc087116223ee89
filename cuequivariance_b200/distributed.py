"""Receiver-range sharding of a channelwise tensor product over the GPUs of one node.

Edges are independent units; the only couplings are the reduction over the edges of a
receiver (made rank-local by giving every rank a contiguous range of receivers and exactly
the edges that point at them) and the gather of sender rows (which needs the other ranks'
node features).  Per step there is therefore one exchange each way:

* forward : all-gather of the node features (each rank contributes its receiver range);
* backward: every rank holds a partial gradient for all nodes (scatter by sender), which a
  reduce-scatter sums back onto the owner ranges.

The reference has no multi-GPU code at all; this is the partition its documentation leaves
to the user (cuequivariance_jax/segmented_polynomials/segmented_polynomial.py:157-162).
One process per GPU, `torch.distributed` (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(num_nodes: int, world: int, rank: int) -> Tuple[int, int]:
    """Receiver range ``[lo, hi)`` owned by ``rank``; ranges are equal (``num_nodes`` must be
    divisible by ``world`` so that the collectives move equal blocks)."""
    if num_nodes % world:
        raise ValueError(f"the number of nodes ({num_nodes}) must be divisible by the number of ranks ({world})")
    per = num_nodes // world
    return rank * per, (rank + 1) * per


def shard_edges(receivers: torch.Tensor, num_nodes: int, world: int, rank: int) -> Tuple[int, int]:
    """Slice ``[e_lo, e_hi)`` of a receiver-sorted edge list that belongs to ``rank``.
    Raises if the list is not sorted (checked on the host before any collective)."""
    if receivers.numel() > 1 and not bool((receivers[1:] >= receivers[:-1]).all()):
        raise ValueError("edges must be sorted by receiver before sharding")
    lo, hi = shard_bounds(num_nodes, world, rank)
    b = torch.tensor([lo, hi], dtype=receivers.dtype, device=receivers.device)
    e = torch.searchsorted(receivers.contiguous(), b)
    return int(e[0]), int(e[1])


def exchange_group_options(max_ctas: Optional[int] = None):
    """NCCL options for the group that carries the node-feature exchange.

    The channelwise launches fill every SM, and thread blocks of a collective issued on a
    normal-priority stream only become resident when the running launch drains, which
    serialises each block's transfer behind the previous launch instead of overlapping it.
    A high-priority stream lets the collective's few blocks in as soon as any block of the
    compute kernel retires; ``max_ctas`` optionally bounds how many SMs it takes away
    (measured on 8 B200s, ms per config-3 step: default stream 3.02; high priority 2.77;
    high priority capped at 32 / 16 / 8 blocks 2.77 / 3.03 / 3.78)."""
    opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
    if max_ctas:
        opts.config.max_ctas = int(max_ctas)
    return opts


def new_exchange_group(ranks=None, max_ctas: Optional[int] = None):
    """A process group for :class:`ReceiverShardedChannelWise` with the options above
    (collective on every rank, like ``torch.distributed.new_group``)."""
    return dist.new_group(ranks=ranks, backend="nccl", pg_options=exchange_group_options(max_ctas))


class _AllGatherRows(torch.autograd.Function):
    """``[n_local, d] -> [n_local * world, d]``; the adjoint is a sum reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = torch.empty((x.shape[0] * world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        world = dist.get_world_size(ctx.group)
        rows = g.shape[0] // world
        g = g.contiguous()
        if g.is_cuda:
            out = torch.empty((rows,) + tuple(g.shape[1:]), dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.SUM, group=ctx.group)
            return out, None
        # CPU backends (gloo) have no reduce-scatter: all-reduce, then keep the owned rows
        g = g.clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        r = dist.get_rank(ctx.group)
        return g[r * rows : (r + 1) * rows].clone(), None


def all_gather_rows(x: torch.Tensor, group=None) -> torch.Tensor:
    return _AllGatherRows.apply(x, group)


BUNDLES = 0   # exchanges per direction in the pipelined path (0: one per irrep, 1: one collective, 2: two bundles)


class _PipelinedShardedChannelwise(torch.autograd.Function):
    """Sharded channelwise product with the node-feature exchange pipelined against the
    per-irrep kernel launches.

    Forward : the node features are all-gathered in bundles of consecutive irrep blocks
              (asynchronous NCCL calls, smallest first); the launches of a bundle only wait for
              that bundle, so every transfer but the first hides behind earlier launches.
    Backward: launches run largest irrep first; as soon as the launches of a bundle have produced
              their part of the node-feature gradient, its reduce-scatter starts and overlaps
              the next launches; the last (smallest) bundle is the only exposed transfer.
    First-order only (differentiating the result again is not supported on this path)."""

    @staticmethod
    def _bundles(plan):
        """Consecutive irrep blocks exchanged together: ``[(first group, last group + 1, column
        offset, width)]``.  Default: one exchange per irrep block.  Measured on 8 B200s (config 3,
        ms per step): one per irrep 2.77, two bundles (the two small leading blocks, then the
        rest) 2.87 - although every collective costs 0.13-0.2 ms of latency at 8 ranks, the finer
        pipeline still wins."""
        groups = plan.groups
        n = len(groups)
        if BUNDLES == 0 or BUNDLES >= n:
            cuts = list(range(n + 1))
        elif BUNDLES == 1 or n < 2:
            cuts = [0, n]
        else:
            cuts = [0, max(1, n // 2), n]
        out = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            off = groups[a]["x1_off"]
            end = groups[b - 1]["x1_off"] + groups[b - 1]["x1_width"]
            if any(groups[i]["x1_off"] + groups[i]["x1_width"] != groups[i + 1]["x1_off"] for i in range(a, b - 1)):
                return [(i, i + 1, groups[i]["x1_off"], groups[i]["x1_width"]) for i in range(n)]   # blocks not adjacent: one each
            out.append((a, b, off, end - off))
        return out

    @staticmethod
    def forward(ctx, handler, group, x1_local, x2, weight, senders, receivers_local):
        from .channelwise import _CSR

        plan = handler.plan
        world = dist.get_world_size(group)
        n_local = x1_local.shape[0]
        dev = x1_local.device
        mul_ir = True
        common = dict(x1_mul_ir=mul_ir, senders=_CSR.int32(senders))
        order, rowptr = _CSR.get(receivers_local, n_local)
        csr = (order, rowptr, n_local)
        bundles = _PipelinedShardedChannelwise._bundles(plan)
        wide, works = [], []
        for (a, b, off, width) in bundles:  # irrep blocks in ascending size
            loc = x1_local[:, off : off + width].contiguous()
            full = torch.empty((n_local * world, width), dtype=loc.dtype, device=dev)
            works.append(dist.all_gather_into_tensor(full, loc, group=group, async_op=True))
            wide.append(full)
        out = torch.empty((n_local, plan.row_sizes[3]), dtype=torch.float32, device=dev)
        for bi, (a, b, off, width) in enumerate(bundles):
            works[bi].wait()
            for gi in range(a, b):
                g = plan.groups[gi]
                block = wide[bi][:, g["x1_off"] - off : g["x1_off"] - off + g["x1_width"]]
                handler.launch_forward_group(gi, common, csr, mul_ir, weight, block, x2, out)
        ctx.handler, ctx.group, ctx.common, ctx.csr, ctx.bundles = handler, group, common, csr, bundles
        ctx.save_for_backward(weight, x2, *wide)
        ctx.n_local = n_local
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gout):
        handler, group, common, csr, bundles = ctx.handler, ctx.group, ctx.common, ctx.csr, ctx.bundles
        plan = handler.plan
        weight, x2, *wide = ctx.saved_tensors
        gout = gout.contiguous()
        need_x1, need_x2, need_w = ctx.needs_input_grad[2], ctx.needs_input_grad[3], ctx.needs_input_grad[4]
        gw = torch.empty_like(weight) if need_w else None
        gx2 = torch.zeros_like(x2) if need_x2 else None
        pieces, works = {}, []
        for bi in reversed(range(len(bundles))):  # largest blocks first
            a, b, off, width = bundles[bi]
            gwide = torch.zeros_like(wide[bi]) if need_x1 else None
            for gi in reversed(range(a, b)):
                g = plan.groups[gi]
                lo = g["x1_off"] - off
                block = wide[bi][:, lo : lo + g["x1_width"]]
                gblock = gwide[:, lo : lo + g["x1_width"]] if need_x1 else None
                handler.launch_backward_group(gi, common, csr, True, weight, block, x2, gout, gw, gblock, gx2)
            if need_x1:
                mine = torch.empty((ctx.n_local, width), dtype=gwide.dtype, device=gwide.device)
                works.append(dist.reduce_scatter_tensor(mine, gwide, op=dist.ReduceOp.SUM, group=group, async_op=True))
                pieces[bi] = mine
        gx1 = None
        if need_x1:
            for wk in works:
                wk.wait()
            gx1 = torch.empty((ctx.n_local, plan.row_sizes[1]), dtype=torch.float32, device=gout.device)
            for bi, (a, b, off, width) in enumerate(bundles):
                gx1[:, off : off + width] = pieces[bi]
        return None, None, gx1, gx2, gw, None, None


class ReceiverShardedChannelWise(torch.nn.Module):
    """``forward(x1_local, x2, weight, senders, receivers_local)``.

    ``x1_local``: this rank's rows of the node features (its receiver range);
    ``x2``/``weight``/``senders``/``receivers_local``: this rank's edges, senders as GLOBAL
    node ids, receivers relative to the start of the rank's range.  Returns this rank's
    rows of the output.  With ``group=None`` (one process) it is the plain fused call.
    """

    def __init__(self, tp: torch.nn.Module, group=None, pipelined: bool = True):
        super().__init__()
        self.tp = tp
        self.group = group
        self.pipelined = pipelined

    def _handler(self, x1_local, x2, weight):
        """The specialised-kernel handler if the pipelined path applies (float32, mul_ir
        layouts, per-edge weights, one launch per irrep of x1), else None."""
        if not self.pipelined or not x1_local.is_cuda or x1_local.dtype != torch.float32:
            return None
        if x2.dtype != torch.float32 or weight.dtype != torch.float32 or weight.shape[0] != x2.shape[0]:
            return None
        prog = self.tp.f._program(torch.float32)
        special = getattr(prog, "_special", None)
        lay = getattr(self.tp, "_layouts", {})
        if special is None or not hasattr(special, "launch_forward_group") or 1 not in lay or 3 not in lay:
            return None
        offs = [g["x1_off"] for g in special.plan.groups]
        if len(set(offs)) != len(offs):
            return None
        return special

    def forward(self, x1_local, x2, weight, senders, receivers_local):
        n_local = x1_local.shape[0]
        if self.group is None:
            return self.tp(x1_local, x2, weight, indices_1=senders, indices_out=receivers_local, size_out=n_local)
        handler = self._handler(x1_local, x2, weight)
        if handler is not None:
            return _PipelinedShardedChannelwise.apply(handler, self.group, x1_local, x2.contiguous(), weight.contiguous(),
                                                      senders, receivers_local)
        x1 = all_gather_rows(x1_local, self.group)
        return self.tp(x1, x2, weight, indices_1=senders, indices_out=receivers_local, size_out=n_local)
