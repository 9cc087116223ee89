"""CPU tests (gloo, world size 2) of the receiver-range sharding logic: edge slicing, the
differentiable all-gather of node features (whose adjoint is the reduce-scatter of their
gradient), and the host-side failure paths (unsorted edges, indivisible node counts)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cuequivariance_b200.distributed import all_gather_rows, shard_bounds, shard_edges

        torch.manual_seed(0)
        N, E, D = 8, 40, 5
        x = torch.randn(N, D, dtype=torch.float64)
        receivers = torch.sort(torch.randint(0, N, (E,))).values
        senders = torch.randint(0, N, (E,))
        wgt = torch.randn(E, D, dtype=torch.float64)
        lo, hi = shard_bounds(N, world, rank)
        e0, e1 = shard_edges(receivers, N, world, rank)
        assert bool(((receivers[e0:e1] >= lo) & (receivers[e0:e1] < hi)).all())
        # sharded "message passing": out[r] = sum_e w[e] * x[sender[e]] over this rank's edges
        x_local = x[lo:hi].clone().requires_grad_(True)
        full = all_gather_rows(x_local)
        assert torch.equal(full.detach(), x)
        msg = wgt[e0:e1] * full[senders[e0:e1]]
        out = torch.zeros(hi - lo, D, dtype=torch.float64).index_add(0, receivers[e0:e1] - lo, msg)
        cot = torch.arange(N * D, dtype=torch.float64).reshape(N, D)
        (out * cot[lo:hi]).sum().backward()
        # single-process reference
        xr = x.clone().requires_grad_(True)
        ref = torch.zeros(N, D, dtype=torch.float64).index_add(0, receivers, wgt * xr[senders])
        (ref * cot).sum().backward()
        ok_out = torch.allclose(out, ref[lo:hi].detach())
        ok_grad = torch.allclose(x_local.grad, xr.grad[lo:hi])
        results[rank] = (ok_out, ok_grad, e1 - e0)
    finally:
        dist.destroy_process_group()


def test_sharded_gather_and_gradient_exchange_world2():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    assert all(r[0] and r[1] for r in results.values())
    assert sum(r[2] for r in results.values()) == 40


def test_shard_helpers_reject_bad_input():
    from cuequivariance_b200.distributed import shard_bounds, shard_edges

    with pytest.raises(ValueError, match="divisible"):
        shard_bounds(10, 4, 0)
    with pytest.raises(ValueError, match="sorted"):
        shard_edges(torch.tensor([3, 1, 2]), 4, 2, 0)
    assert shard_bounds(8, 4, 3) == (6, 8)
    assert shard_edges(torch.tensor([0, 0, 1, 3, 3, 3]), 4, 2, 1) == (3, 6)


def test_exchange_bundles_cover_every_block_once():
    """Host logic of the pipelined path: irrep blocks are grouped into bundles of adjacent column ranges."""
    from types import SimpleNamespace

    from cuequivariance_b200 import distributed
    from cuequivariance_b200.distributed import _PipelinedShardedChannelwise as P

    groups = [dict(x1_off=0, x1_width=128), dict(x1_off=128, x1_width=384), dict(x1_off=512, x1_width=640), dict(x1_off=1152, x1_width=896)]
    plan = SimpleNamespace(groups=groups)
    old = distributed.BUNDLES
    try:
        distributed.BUNDLES = 2
        assert P._bundles(plan) == [(0, 2, 0, 512), (2, 4, 512, 1536)]
        distributed.BUNDLES = 1
        assert P._bundles(plan) == [(0, 4, 0, 2048)]
        for per_irrep in (0, 4):
            distributed.BUNDLES = per_irrep
            assert P._bundles(plan) == [(0, 1, 0, 128), (1, 2, 128, 384), (2, 3, 512, 640), (3, 4, 1152, 896)]
        distributed.BUNDLES = 2
        gap = [dict(x1_off=0, x1_width=128), dict(x1_off=256, x1_width=128)]     # not adjacent: one exchange each
        assert P._bundles(SimpleNamespace(groups=gap)) == [(0, 1, 0, 128), (1, 2, 256, 128)]
    finally:
        distributed.BUNDLES = old


def _board_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import random
        import time

        from cuequivariance_b200.distributed import HandshakeBoard

        board = HandshakeBoard()
        rng = random.Random(rank)
        ok = True
        for k in range(40):                       # the peer-exchange protocol: publish, then wait for everybody
            time.sleep(rng.random() * 0.003)
            board.publish(k + 1)
            for q in range(world):
                if q != rank:
                    board.wait_for(q, k + 1, 20.0)
                    ok = ok and int(board.counters[q]) >= k + 1        # nobody is let through early
                    ok = ok and int(board.counters[q]) <= k + 2        # and nobody runs more than one hand-shake ahead
        dist.barrier()
        # a rank that never arrives ends the wait with an error on the host, it does not hang
        if rank == 0:
            t0 = time.monotonic()
            try:
                board.wait_for(1, 1000, 0.2)
                ok = False
            except RuntimeError as e:
                ok = ok and "did not reach" in str(e) and time.monotonic() - t0 < 5.0
        dist.barrier()
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_handshake_board_world2():
    """The host half of the kernel-free hand-shake of the peer exchange (counter page in shared memory)."""
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_board_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world and all(results.values())
