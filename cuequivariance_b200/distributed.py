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


class ReceiverShardedChannelWise(torch.nn.Module):
    """``forward(x1_local, x2, weight, senders, receivers_local)``.

    ``x1_local``: this rank's rows of the node features (its receiver range);
    ``x2``/``weight``/``senders``/``receivers_local``: this rank's edges, senders as GLOBAL
    node ids, receivers relative to the start of the rank's range.  Returns this rank's
    rows of the output.  With ``group=None`` (one process) it is the plain fused call.
    """

    def __init__(self, tp: torch.nn.Module, group=None):
        super().__init__()
        self.tp = tp
        self.group = group

    def forward(self, x1_local, x2, weight, senders, receivers_local):
        n_local = x1_local.shape[0]
        x1 = x1_local if self.group is None else all_gather_rows(x1_local, self.group)
        return self.tp(x1, x2, weight, indices_1=senders, indices_out=receivers_local, size_out=n_local)
