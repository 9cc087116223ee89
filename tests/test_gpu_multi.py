"""Two-GPU parity of the receiver-sharded channelwise product against the single-GPU call: the
pipelined path with the rows pushed into peer-mapped buffers (by the copy engines and by the push
kernel), the same path with NCCL all-gather / reduce-scatter, and the plain path.  Every variant runs three steps in a
row (the exchange buffers are reused from step to step).  Skipped on boxes with fewer than two
GPUs."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import cuequivariance_b200 as cb
        from cuequivariance_b200 import distributed
        from cuequivariance_b200.distributed import ReceiverShardedChannelWise, shard_bounds, shard_edges

        s1 = "32x0e+32x1o+32x2e+32x3o"
        filt = ["0e", "1o", "2e", "3o"]
        tp = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", filt, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
        gen = torch.Generator(device=dev).manual_seed(9)  # same seed on every rank: identical global data
        E, N = 4000, 64
        x1 = torch.randn(N, tp.irreps_in1.dim, generator=gen, device=dev)
        x2 = torch.randn(E, 16, generator=gen, device=dev)
        w = torch.randn(E, tp.weight_numel, generator=gen, device=dev)
        snd = torch.randint(0, N, (E,), generator=gen, device=dev, dtype=torch.int32)
        rcv = torch.sort(torch.randint(0, N, (E,), generator=gen, device=dev, dtype=torch.int32)).values
        cot = torch.randn(N, tp.irreps_out.dim, generator=gen, device=dev)

        def grads(fn, a, b, c, ct):
            a, b, c = (t.clone().requires_grad_(True) for t in (a, b, c))
            out = fn(a, b, c)
            return [out.detach()] + list(torch.autograd.grad((out * ct).sum(), (a, b, c)))

        ref = grads(lambda a, b, c: tp(a, b, c, indices_1=snd, indices_out=rcv, size_out=N), x1, x2, w, cot)
        lo, hi = shard_bounds(N, world, rank)
        e0, e1 = shard_edges(rcv, N, world, rank)
        ok = True
        for pipelined, exchange, push, shake in ((True, "peer_copy", "memcpy", "events"), (True, "peer_copy", "kernel", "events"),
                                                 (True, "peer_copy", "memcpy", "nccl"), (True, "nccl", "", ""), (False, "nccl", "", "")):
            distributed.EXCHANGE, distributed.PUSH_MODE = exchange, push or distributed.PUSH_MODE
            if shake:
                distributed.HANDSHAKE = shake
                distributed._EXCHANGES.clear()      # the hand-shake kind is fixed when an exchange is set up
            op = ReceiverShardedChannelWise(tp, group=dist.group.WORLD, pipelined=pipelined)
            for step in range(3):
                scale_in = 1.0 + step    # different data every step: a stale buffer would show
                got = grads(lambda a, b, c: op(a, b, c, snd[e0:e1].contiguous(), (rcv[e0:e1] - lo).contiguous()),
                            scale_in * x1[lo:hi], x2[e0:e1], w[e0:e1], cot[lo:hi])
                want = [scale_in * ref[0][lo:hi], ref[1][lo:hi], scale_in * ref[2][e0:e1], scale_in * ref[3][e0:e1]]
                for g_, w_ in zip(got, want):
                    scale = max(1.0, float(w_.abs().max()))
                    ok = ok and bool(((g_ - w_).abs() <= 1e-4 * w_.abs() + 2e-5 * scale).all())
            if pipelined and exchange == "peer_copy":
                ok = ok and any(bool(v) for v in distributed._EXCHANGES.values())   # the peer-copy exchange was really set up
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_receiver_sharded_channelwise_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world and all(results.values())


def _one_process_two_devices(results):
    """Child process: the same kernels on cuda:0 and then on cuda:1 of ONE process.  Every launcher raises the
    dynamic shared-memory limit of its kernel once per device; a process-wide flag would leave the second device
    at 48 KB and its launch would fail."""
    sys.path.insert(0, ROOT)
    import cuequivariance_b200 as cb
    from cuequivariance_b200 import _lib
    from cuequivariance_b200.dense import linear_f32x3

    s1 = "+".join(f"128x{ir}" for ir in ("0e", "1o", "2e", "3o"))
    filt = ["0e", "1o", "2e", "3o"]
    tp = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", filt, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    gen = torch.Generator().manual_seed(5)
    E, N = 600, 40
    x1, x2, w = torch.randn(N, tp.irreps_in1.dim, generator=gen), torch.randn(E, 16, generator=gen), torch.randn(E, tp.weight_numel, generator=gen)
    snd = torch.randint(0, N, (E,), generator=gen, dtype=torch.int32)
    rcv = torch.sort(torch.randint(0, N, (E,), generator=gen, dtype=torch.int32)).values
    cot = torch.randn(N, tp.irreps_out.dim, generator=gen)
    xa, wa = torch.randn(512, 64, generator=gen), torch.randn(256, 64, generator=gen)
    outs = []
    for d in ("cuda:0", "cuda:1"):
        a, b, c = (t.to(d).requires_grad_(True) for t in (x1, x2, w))
        out = tp(a, b, c, indices_1=snd.to(d), indices_out=rcv.to(d), size_out=N)      # backward of the l >= 2 groups: > 48 KB
        g = torch.autograd.grad((out * cot.to(d)).sum(), (a, b, c))
        xl, wl = xa.to(d).requires_grad_(True), wa.to(d).requires_grad_(True)
        y = linear_f32x3(xl, wl)                                                       # tcgen05 kernels: > 100 KB
        gy = torch.autograd.grad(y.sum(), (xl, wl))
        torch.cuda.synchronize(d)
        _lib.check_status()
        outs.append([t.detach().cpu() for t in (out, *g, y, *gy)])
    ok = True
    for p, q in zip(*outs):
        ok = ok and bool((p - q).abs().max() <= 1e-4 * max(1.0, float(p.abs().max())))   # reduction order differs from run to run
    results["ok"] = ok


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_drives_two_devices():
    import torch.multiprocessing as mp

    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_one_process_two_devices_entry, args=(results,), nprocs=1, join=True)
    assert results.get("ok") is True


def _one_process_two_devices_entry(_index, results):
    _one_process_two_devices(results)
