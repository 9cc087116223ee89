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


import os as _os

_DIAG_SKIP_COPY = bool(_os.environ.get("CUEQ_DIAG_SKIP_COPY"))
_DIAG_SKIP_HANDSHAKE = bool(_os.environ.get("CUEQ_DIAG_SKIP_HANDSHAKE"))
PUSH_BLOCKS = int(_os.environ.get("CUEQ_PUSH_BLOCKS", "4"))      # thread blocks per (peer, irrep block) piece of the push kernel
PUSH_MODE = _os.environ.get("CUEQ_PUSH_MODE", "memcpy")   # "memcpy": one cudaMemcpyAsync per piece (copy engines); "kernel": the push kernel
HANDSHAKE = _os.environ.get("CUEQ_HANDSHAKE", "events")   # peer exchange: "events" (interprocess CUDA events, no kernel) or "nccl" (one-element all-reduce)
HANDSHAKE_TIMEOUT_S = 60.0
EXCHANGE = _os.environ.get("CUEQ_EXCHANGE", "nccl")       # how the pipelined path moves node rows between ranks: "nccl" or "peer_copy"


class HandshakeBoard:
    """One counter per rank in a page of host memory shared by the ranks of one node.

    ``publish(k)`` sets this rank's counter; ``wait_for(q, k)`` polls rank ``q``'s counter on the host until it
    has reached ``k`` (bounded: raises after ``timeout`` seconds, e.g. when rank ``q`` has died).  The page is a
    small file in shared memory that every rank maps; rank 0 removes its name as soon as everybody has it open
    (the mappings stay valid), so nothing is left behind whatever happens later.  Needs no GPU."""

    def __init__(self, group=None):
        import os
        import tempfile

        import numpy as np

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        path = [None]
        if self.rank == 0:
            fd, path[0] = tempfile.mkstemp(prefix="cueq_b200_handshake_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
            os.write(fd, bytes(8 * self.world))
            os.close(fd)
        dist.broadcast_object_list(path, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self.counters = np.memmap(path[0], dtype=np.int64, mode="r+", shape=(self.world,))
        dist.barrier(group=group)
        if self.rank == 0:
            os.unlink(path[0])

    def publish(self, k: int) -> None:
        self.counters[self.rank] = k

    def wait_for(self, q: int, k: int, timeout: float) -> None:
        import time

        deadline = time.monotonic() + timeout
        while self.counters[q] < k:
            if time.monotonic() > deadline:
                raise RuntimeError(f"rank {q} did not reach hand-shake {k - 1} within {timeout} s (its counter is {int(self.counters[q])})")


class PeerExchange:
    """Node-feature exchange between the ranks of one node without taking SMs from the kernels.

    The channelwise launches fill every SM, so a collective's thread blocks compete with them (and
    wait for a free slot before a transfer can even start).  Here every rank owns a receive buffer
    that the other ranks have mapped through CUDA IPC, and a rank *pushes* its contribution into
    each peer's buffer with this library's push kernel (``csrc/peer_copy.cu``: 16-byte stores over
    NVLink, one launch per irrep block covering all peers, a few thread blocks per peer) on a
    high-priority side stream.  Why a kernel and why pushing, measured on two B200s: a
    ``cudaMemcpyAsync`` into IPC-mapped peer memory blocked the issuing host thread for the length
    of the copy (1.3 ms per call, the host fell behind the device), and a transfer that reads from
    the peer ran at 24 GB/s where the same transfer written to the peer ran at 650 GB/s.  Plain
    stores only: no multicast, no TMA.  What still needs a collective is the hand-shake "everybody's rows have
    landed" before a block is used and "everybody is done with the buffer" before it is written
    again: a one-element all-reduce on a high-priority stream.  A rank that dies leaves the others
    in that collective, which the process-group time-out ends on the host; nothing on the device
    waits on a flag.

    Receive buffers (float32): ``full[l]`` = irrep block ``l`` of the node features of ALL ranks
    ``[n_local * world, width_l]`` (forward); ``stage[l]`` = the other ranks' partial gradients of
    this rank's rows ``[world, n_local, width_l]`` (backward; slot ``r`` is written by rank ``r``).
    """

    def __init__(self, group, n_local: int, widths, device):
        import ctypes as C

        from . import _lib

        self.group, self.n_local, self.widths = group, n_local, list(widths)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.device = device
        n_all = n_local * self.world
        sizes = [n_all * w for w in self.widths] + [n_all * w for w in self.widths]
        self.offsets = [0]
        for sz in sizes:
            self.offsets.append(self.offsets[-1] + (sz + 63) // 64 * 64)
        self.flat = torch.empty(self.offsets[-1], dtype=torch.float32, device=device)
        # every rank exports its buffer; every other rank maps it for ITS OWN device (see csrc/peer_copy.cu)
        handle, offset = C.create_string_buffer(64), C.c_int64(0)
        with torch.cuda.device(device):
            _lib.check(_lib.lib().cueq_b200_ipc_export(C.c_void_p(self.flat.data_ptr()), handle, C.byref(offset)))
        handles = [None] * self.world
        dist.all_gather_object(handles, (bytes(handle.raw), int(offset.value)), group=group)
        self.peers, self._mapped = [], []
        for r, (raw, off) in enumerate(handles):
            if r == self.rank:
                self.peers.append(self.flat)
                continue
            base = C.c_void_p()
            with torch.cuda.device(device):
                _lib.check(_lib.lib().cueq_b200_ipc_open(C.create_string_buffer(raw, 64), C.byref(base)))
            self._mapped.append(base)
            self.peers.append(_as_tensor(base.value + off, self.flat.numel(), device))
        nb = len(self.widths)
        self.full = [self._view(self.flat, l, n_all, self.widths[l]) for l in range(nb)]
        self.stage = [self._view(self.flat, nb + l, n_all, self.widths[l]).view(self.world, n_local, self.widths[l]) for l in range(nb)]
        self.x = [torch.empty((n_local, w), dtype=torch.float32, device=device) for w in self.widths]   # contiguous send copies
        self.copy_streams = [torch.cuda.Stream(device=device, priority=-1) for _ in range(max(1, self.world - 1))]
        self.exch = torch.cuda.Stream(device=device, priority=-1)
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.free = None                  # event: every rank is done with the receive buffers of the previous pass
        self.handshake_mode = HANDSHAKE
        if self.handshake_mode == "events":
            self._setup_event_handshake()

    # -- hand-shake without a kernel -----------------------------------------------------------------
    #
    # A collective needs thread blocks, and while a channelwise launch holds every register of every SM its
    # blocks are not scheduled before that launch drains - the hand-shake then costs as long as the kernel
    # it was meant to overlap.  Interprocess CUDA events need no SM: rank r records event E[r][k % S] on its
    # exchange stream and the others make their exchange streams wait for it.  A stream wait captures the
    # event's latest record *at the time of the call*, so a waiter must not call before the record has been
    # issued: every rank publishes the number of records it has issued in a page of host shared memory
    # (`HandshakeBoard`) and a waiter polls that counter (on the host, bounded) first.  An event slot is recorded again S hand-shakes
    # later; by then every rank has issued its waits for the earlier record, because nobody starts hand-shake
    # k + 1 before everybody has published hand-shake k.
    _SLOTS = 8

    def _setup_event_handshake(self):
        dev = self.device
        with torch.cuda.device(dev):
            self._ev_local = [torch.cuda.Event(enable_timing=False, interprocess=True) for _ in range(self._SLOTS)]
            for ev in self._ev_local:
                ev.record(self.exch)               # an event must have been recorded before its handle is exported
            handles = [ev.ipc_handle() for ev in self._ev_local]
        self._board = HandshakeBoard(self.group)
        all_handles = [None] * self.world
        dist.all_gather_object(all_handles, handles, group=self.group)
        self._ev_peer = []
        for r, hs in enumerate(all_handles):
            if r == self.rank:
                self._ev_peer.append(self._ev_local)
            else:
                self._ev_peer.append([torch.cuda.Event.from_ipc_handle(dev, h) for h in hs])
        self._count = 0
        dist.barrier(group=self.group)             # nobody polls a counter page that does not exist yet

    def _event_handshake(self, s):
        k = self._count
        slot = k % self._SLOTS
        self._ev_local[slot].record(s)
        self._board.publish(k + 1)                 # the record has been issued: peers may issue their waits
        for q in range(self.world):
            if q != self.rank:
                self._board.wait_for(q, k + 1, HANDSHAKE_TIMEOUT_S)
                s.wait_event(self._ev_peer[q][slot])
        self._count = k + 1

    def _view(self, flat, slot, rows, width):
        return flat[self.offsets[slot] : self.offsets[slot] + rows * width].view(rows, width)

    def peer_full_rows(self, q, l):
        """Where this rank's rows of block ``l`` go inside rank ``q``'s gathered block."""
        full = self._view(self.peers[q], l, self.n_local * self.world, self.widths[l])
        return full[self.rank * self.n_local : (self.rank + 1) * self.n_local]

    def peer_stage_slot(self, q, l):
        """This rank's slot in rank ``q``'s staging area for block ``l``."""
        st = self._view(self.peers[q], len(self.widths) + l, self.n_local * self.world, self.widths[l])
        return st[self.rank * self.n_local : (self.rank + 1) * self.n_local]

    def handshake(self, after_events=()):
        """An event that completes once every rank has reached this point (each rank's collective
        starts only after the events it was given)."""
        s = self.exch
        for ev in after_events:
            s.wait_event(ev)
        if self.handshake_mode == "events":
            self._event_handshake(s)
        elif not _DIAG_SKIP_HANDSHAKE:
            with torch.cuda.stream(s):
                dist.all_reduce(self.flag, group=self.group)
        ev = torch.cuda.Event()
        ev.record(s)
        return ev

    def push(self, pieces, after_events):
        """``pieces`` = [(dst, src)]: ``dst`` a peer's buffer, ``src`` local, both contiguous and of equal size.  One
        launch of the push kernel per eight pieces on the exchange's copy stream; returns the completion event."""
        import ctypes as C

        from . import _lib

        s = self.copy_streams[0]
        for ev in after_events:
            if ev is not None:
                s.wait_event(ev)
        if PUSH_MODE == "memcpy" and not _DIAG_SKIP_COPY:   # copy engines instead of the push kernel
            # one stream per peer: the copies of a block go out over all links at once instead of one after the other
            # (a single copy engine does not fill a link, and a single stream uses a single engine at a time)
            start = torch.cuda.Event()
            start.record(s)
            used = []
            with torch.cuda.device(self.device):
                for k, (dst, src) in enumerate(pieces):
                    sk = self.copy_streams[k % len(self.copy_streams)]
                    if sk is not s and sk not in used:
                        sk.wait_event(start)
                        used.append(sk)
                    _lib.check(_lib.lib().cueq_b200_copy_async(C.c_void_p(dst.data_ptr()), C.c_void_p(src.data_ptr()),
                                                               C.c_size_t(src.numel() * src.element_size()), C.c_void_p(sk.cuda_stream)))
            for sk in used:                                  # the returned event covers every stream
                e = torch.cuda.Event()
                e.record(sk)
                s.wait_event(e)
            pieces = []
        for i in range(0, len(pieces), 8):
            a = _lib.PushArgs()
            chunk = pieces[i : i + 8]
            for k, (dst, src) in enumerate(chunk):
                a.dst[k], a.src[k], a.bytes[k] = dst.data_ptr(), src.data_ptr(), src.numel() * src.element_size()
            a.num_pieces, a.blocks_per_piece = len(chunk), PUSH_BLOCKS
            if not _DIAG_SKIP_COPY:
                with torch.cuda.device(self.device):
                    _lib.check(_lib.lib().cueq_b200_push(C.byref(a), C.c_void_p(s.cuda_stream)))
        ev = torch.cuda.Event()
        ev.record(s)
        return ev


class _RawDeviceArray:
    """Exposes a raw device pointer through the CUDA array interface so that torch can wrap it without a copy."""

    def __init__(self, ptr: int, numel: int):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def _as_tensor(ptr: int, numel: int, device) -> torch.Tensor:
    return torch.as_tensor(_RawDeviceArray(ptr, numel), device=device)


_EXCHANGES: dict = {}


def _exchange_for(group, n_local, widths, device):
    key = (id(group), n_local, tuple(widths), device)
    ex = _EXCHANGES.get(key)
    if ex is None:
        try:
            ex = PeerExchange(group, n_local, widths, device)
        except Exception as e:  # no peer access between the GPUs (or IPC not permitted): NCCL carries the rows instead
            import warnings

            warnings.warn(f"peer-mapped exchange buffers are not available ({type(e).__name__}: {e}); using NCCL collectives")
            ex = False
        # every rank must take the same route: the exchange works only if it was set up everywhere
        ok = torch.tensor([1.0 if ex else 0.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if float(ok[0]) == 0.0:
            ex = False
        _EXCHANGES[key] = ex
    return ex or None


class _PeerCopyShardedChannelwise(torch.autograd.Function):
    """Same computation as `_PipelinedShardedChannelwise` with the rows moved by `PeerExchange`:
    forward pushes this rank's node rows into every peer's gathered blocks (smallest irrep first) and
    launches a block's kernel once all ranks' rows of it have landed; backward lets every group launch
    reduce into a local partial-gradient block and pushes each peer's rows of it into that peer's staging
    slot as soon as the launch is done, the owner adds the slots up.  First-order only.

    The gathered blocks live in the exchange's persistent receive buffers.  With ``keep`` they are cloned for
    the backward pass; without, the backward pass reads the buffers themselves, which is valid as long as the
    backward of a forward runs before the next forward of the same module (the usual training step)."""

    @staticmethod
    def forward(ctx, handler, ex, keep, x1_local, x2, weight, senders, receivers_local):
        from .channelwise import _CSR

        plan = handler.plan
        world, rank, n_local = ex.world, ex.rank, ex.n_local
        dev = x1_local.device
        main = torch.cuda.current_stream(dev)
        common = dict(x1_mul_ir=True, senders=_CSR.int32(senders))
        order, rowptr = _CSR.get(receivers_local, n_local)
        csr = (order, rowptr, n_local)
        groups = plan.groups
        for l, g in enumerate(groups):
            ex.x[l].copy_(x1_local[:, g["x1_off"] : g["x1_off"] + g["x1_width"]])
        written = torch.cuda.Event()
        written.record(main)
        ready = []
        for l in range(len(groups)):
            pieces = [(ex.peer_full_rows((rank + k) % world, l), ex.x[l]) for k in range(1, world)]
            ready.append(ex.handshake([ex.push(pieces, (written, ex.free))]))
        if ex.free is not None:
            main.wait_event(ex.free)               # this rank's own rows also go into a buffer the last pass may still read
        out = torch.empty((n_local, plan.row_sizes[3]), dtype=torch.float32, device=dev)
        for l, g in enumerate(groups):
            ex.full[l][rank * n_local : (rank + 1) * n_local].copy_(ex.x[l])
            main.wait_event(ready[l])
            handler.launch_forward_group(l, common, csr, True, weight, ex.full[l], x2, out)
        wide = [t.clone() for t in ex.full] if keep else list(ex.full)
        done = torch.cuda.Event()
        done.record(main)
        ex.free = ex.handshake([done])             # superseded by the backward's own if one follows
        ctx.handler, ctx.ex, ctx.common, ctx.csr, ctx.keep = handler, ex, common, csr, keep
        ctx.save_for_backward(weight, x2, *wide)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gout):
        handler, ex, common, csr = ctx.handler, ctx.ex, ctx.common, ctx.csr
        plan = handler.plan
        world, rank, n_local = ex.world, ex.rank, ex.n_local
        weight, x2, *wide = ctx.saved_tensors
        dev = gout.device
        main = torch.cuda.current_stream(dev)
        gout = gout.contiguous()
        need_x1, need_x2, need_w = ctx.needs_input_grad[3], ctx.needs_input_grad[4], ctx.needs_input_grad[5]
        gw = torch.empty_like(weight) if need_w else None
        gx2 = torch.zeros_like(x2) if need_x2 else None
        groups = plan.groups
        partial, ready = {}, {}
        for l in reversed(range(len(groups))):    # largest blocks first: their transfers hide behind the later launches
            gl = torch.zeros((n_local * world, groups[l]["x1_width"]), dtype=torch.float32, device=dev) if need_x1 else None
            handler.launch_backward_group(l, common, csr, True, weight, wide[l], x2, gout, gw, gl, gx2)
            if need_x1:
                done = torch.cuda.Event()
                done.record(main)
                pieces = []
                for k in range(1, world):
                    q = (rank + k) % world
                    pieces.append((ex.peer_stage_slot(q, l), gl[q * n_local : (q + 1) * n_local]))
                ex.stage[l][rank].copy_(gl[rank * n_local : (rank + 1) * n_local])      # this rank's own contribution
                partial[l], ready[l] = gl, ex.handshake([ex.push(pieces, (done,))])
        gx1 = None
        if need_x1:
            gx1 = torch.empty((n_local, plan.row_sizes[1]), dtype=torch.float32, device=dev)
            for l, g in enumerate(groups):
                main.wait_event(ready[l])
                gx1[:, g["x1_off"] : g["x1_off"] + g["x1_width"]] = ex.stage[l].sum(0)
        done = torch.cuda.Event()
        done.record(main)
        ex.free = ex.handshake([done])            # receive buffers (gathered blocks, staging slots) may be rewritten after this
        return None, None, None, gx1, gx2, gw, None, None


class ReceiverShardedChannelWise(torch.nn.Module):
    """``forward(x1_local, x2, weight, senders, receivers_local)``.

    ``x1_local``: this rank's rows of the node features (its receiver range);
    ``x2``/``weight``/``senders``/``receivers_local``: this rank's edges, senders as GLOBAL
    node ids, receivers relative to the start of the rank's range.  Returns this rank's
    rows of the output.  With ``group=None`` (one process) it is the plain fused call.
    """

    def __init__(self, tp: torch.nn.Module, group=None, pipelined: bool = True, keep_gathered: bool = True):
        super().__init__()
        self.tp = tp
        self.group = group
        self.pipelined = pipelined
        # False: the backward pass reads the gathered node features from the exchange's receive buffers instead of a
        # copy; valid when every forward is followed by its backward before the next forward (a training step)
        self.keep_gathered = keep_gathered

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
            if EXCHANGE == "peer_copy" and dist.get_world_size(self.group) > 1:
                ex = _exchange_for(self.group, n_local, [g["x1_width"] for g in handler.plan.groups], x1_local.device)
                if ex is not None:
                    return _PeerCopyShardedChannelwise.apply(handler, ex, self.keep_gathered, x1_local, x2.contiguous(),
                                                             weight.contiguous(), senders, receivers_local)
            return _PipelinedShardedChannelwise.apply(handler, self.group, x1_local, x2.contiguous(), weight.contiguous(),
                                                      senders, receivers_local)
        x1 = all_gather_rows(x1_local, self.group)
        return self.tp(x1, x2, weight, indices_1=senders, indices_out=receivers_local, size_out=n_local)
