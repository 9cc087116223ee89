"""Benchmark of the headline metric: edges/s of the channelwise tensor product, forward +
backward, 1,048,576 edges / 32,768 nodes / 128 channels / lmax 3, float32, on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one forward + one backward (gradients w.r.t. weights, node features and
spherical harmonics) of `ChannelWiseTensorProduct` with gather by sender and scatter-add
to receivers.  Inputs are seeded synthetic tensors with the shapes and distributions of the
named configuration (node features N(0,1); spherical harmonics of random unit vectors;
per-edge weights from a 2-layer radial MLP on Bessel functions of edge lengths uniform in
[0.5, 5]; receivers sorted; senders uniform).  With N > 1 edges are sharded by receiver
range, node features are all-gathered and their gradient reduce-scattered (NCCL).

The JSON line carries: `value` (device-resident inputs, CUDA-event timing, max over
ranks), `e2e` (same step fed from pinned host buffers through the public module API,
including the radial MLP and spherical harmonics that produce the per-edge operands),
`roofline` (dominant kernel, timed live with CUDA events around its launches),
`cpu_baseline` (the CPU oracle on a bounded slice, rank 0, N=1) and `clocks`.
`--impl reference` times the CPU arm alone: the unmodified reference's naive path when it is
staged under `baseline/_ref` (kind "reference"), else the oracle port (kind "port"); same slice.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

E_TOTAL, N_TOTAL, MUL = 1_048_576, 32_768, 128
IRREPS1 = "+".join(f"{MUL}x{ir}" for ir in ("0e", "1o", "2e", "3o"))
IRREPS2 = "0e+1o+2e+3o"
FILTER = ["0e", "1o", "2e", "3o"]
CPU_SAMPLE_EDGES, CPU_SAMPLE_NODES = 16384, 512


# ----------------------------------------------------------------------------------------------
def bessel(r, n=8, rc=5.0):
    import torch

    k = torch.arange(1, n + 1, device=r.device, dtype=r.dtype) * math.pi / rc
    return math.sqrt(2.0 / rc) * torch.sin(k * r[:, None]) / r[:, None]


def make_mlp(weight_numel, device, seed=32):
    import torch

    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(8, 64), torch.nn.SiLU(), torch.nn.Linear(64, weight_numel)).to(device)


class ClockSampler:
    """Samples nvidia-smi clocks/throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
def cpu_oracle_rate(edges=CPU_SAMPLE_EDGES, nodes=CPU_SAMPLE_NODES, repeats=1, warmup=0):
    """Edges/s of the CPU oracle (port of the reference's naive torch path) on a slice of the
    workload: same irreps and channel count, fewer edges and nodes; forward + backward."""
    import torch

    import cuequivariance_b200 as cb
    from oracle import naive

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    e = cb.descriptors.channelwise_tensor_product(IRREPS1, IRREPS2, FILTER)
    b1 = [(m, ir.dim) for m, ir in e.inputs[1].irreps]
    bo = [(m, ir.dim) for m, ir in e.outputs[0].irreps]
    gen = torch.Generator().manual_seed(30)
    x1 = torch.randn(nodes, e.inputs[1].dim, generator=gen)
    vec = torch.nn.functional.normalize(torch.randn(edges, 3, generator=gen), dim=1)
    sh = cb.descriptors.spherical_harmonics("1o", [0, 1, 2, 3])
    x2 = naive.segmented_polynomial(sh.polynomial, [vec])[0]
    w = torch.randn(edges, e.inputs[0].dim, generator=gen)
    snd = torch.randint(0, nodes, (edges,), generator=gen)
    rcv = torch.sort(torch.randint(0, nodes, (edges,), generator=gen)).values
    cot = torch.randn(nodes, e.outputs[0].dim, generator=gen)

    def step():
        xs = [t.clone().requires_grad_(True) for t in (w, x1, x2)]
        (o,) = naive.segmented_polynomial(e.polynomial, [xs[0], naive.transpose_layout(xs[1], b1, True), xs[2]], {1: snd}, {0: nodes}, {0: rcv})
        o = naive.transpose_layout(o, bo, False)
        torch.autograd.grad((o * cot).sum(), xs)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return edges / (sum(times) / len(times)), cores, sum(times) / len(times)


def cpu_reference_rate(edges=CPU_SAMPLE_EDGES, nodes=CPU_SAMPLE_NODES, repeats=1, warmup=0):
    """The same slice through the unmodified reference (its `ChannelWiseTensorProduct` with
    `method="naive"`, the only execution path it has without its closed kernel package), when
    the reference is staged under `baseline/_ref`; returns None otherwise."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import refenv

    if not refenv.available():
        return None
    import torch

    cue, cuet = refenv.activate()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    tp = cuet.ChannelWiseTensorProduct(cue.Irreps("O3", IRREPS1), cue.Irreps("O3", IRREPS2), [cue.O3(l, (-1) ** l) for l in range(4)],
                                       layout=cue.mul_ir, shared_weights=False, internal_weights=False, method="naive")
    sh = cuet.SphericalHarmonics([0, 1, 2, 3], normalize=True, method="naive")
    gen = torch.Generator().manual_seed(30)
    x1 = torch.randn(nodes, tp.irreps_in1.dim, generator=gen)
    x2 = sh(torch.randn(edges, 3, generator=gen)).detach()
    w = torch.randn(edges, tp.weight_numel, generator=gen)
    snd = torch.randint(0, nodes, (edges,), generator=gen)
    rcv = torch.sort(torch.randint(0, nodes, (edges,), generator=gen)).values
    cot = torch.randn(nodes, tp.irreps_out.dim, generator=gen)

    def step():
        xs = [t.clone().requires_grad_(True) for t in (w, x1, x2)]
        o = tp(xs[1], xs[2], xs[0], indices_1=snd, indices_out=rcv, size_out=nodes)
        torch.autograd.grad((o * cot).sum(), xs)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return edges / (sum(times) / len(times)), cores, sum(times) / len(times)


def cpu_baseline(repeats=1, warmup=0):
    """(rate, cores, seconds per step, kind): the reference itself when staged, else the port."""
    try:
        r = cpu_reference_rate(repeats=repeats, warmup=warmup)
    except Exception as ex:  # a broken staging must not take the benchmark down: fall back to the port and say so
        sys.stderr.write(f"reference arm: staged reference failed ({type(ex).__name__}: {ex}); timing the port\n")
        r = None
    if r is not None:
        return r + ("reference",)
    return cpu_oracle_rate(repeats=repeats, warmup=warmup) + ("port",)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rate, cores, sec, kind = cpu_baseline(repeats=args.steps, warmup=args.warmup)
    sample = f"{CPU_SAMPLE_EDGES} edges / {CPU_SAMPLE_NODES} nodes of the same irreps and channel count, fwd+bwd, per step"
    print(json.dumps({
        "impl": "reference", "metric": "edges/s channelwise TP fwd+bwd (1M edges,128ch,lmax3)", "value": rate, "unit": "edges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config 3 shape, CPU slice: " + sample, "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": rate, "unit": "edges/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": rate, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def kernel_source_digest() -> str:
    """SHA-1 over the sources of the channelwise kernels (what a DRAM-traffic capture is valid for)."""
    import hashlib

    h = hashlib.sha1()
    for name in ("cw_kernels.cu", "cw_macros.cuh", "gen_cw_groups.py"):
        with open(os.path.join(ROOT, "cuequivariance_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


# ----------------------------------------------------------------------------------------------
def group_bytes(plan, g, E, n_recv, n_nodes, backward: bool):
    """Algorithmic HBM bytes of one launch of one group: every operand element the launch
    needs, read or written once (gathers counted once per source row)."""
    X = plan.extent * 4
    d1 = {0: 1, 1: 3, 2: 5, 3: 7}
    import cuequivariance_b200._lib as L

    sig = L.lib().cueq_b200_cw_group_signature(g["id"]).decode()
    l1 = int(sig.split(":")[0])
    d3 = sum(2 * int(t.split(".")[1]) + 1 for t in sig.split(":")[1].split(","))
    npath = g["npath"]
    edge = npath * X + 16 * 4 + 8            # weight segments + x2 row + two indices
    b = E * edge + n_nodes * d1[l1] * X      # + the x1 irrep block of every node
    if not backward:
        return b + n_recv * d3 * X           # + output blocks
    return b + n_recv * d3 * X + E * (npath * X + 16 * 4) + n_nodes * d1[l1] * X  # + gw, gx2, gx1


def sharded_parity(tp, out, gx1, x1_l, x2, w, snd_l, rcv_l, cot, N, world, rank, dev):
    """Correctness of the sharded step, checked outside the timed region on a fixed sub-graph against
    single-GPU evaluations of the same module (which the test-suite pins on the CPU oracle):

    * every rank: its first 256 output rows against the plain fused call on the full node table (all of
      those receivers' edges are local to the rank, the node table is all-gathered once for the check);
    * the node-feature gradient rows of nodes [0, 32) (owned by rank 0): edges that send from those nodes
      live on every rank, so each rank contributes its matching edges (weights, harmonics, and the cotangent
      row of each edge's receiver) by all-gather; rank 0 evaluates them unsharded and compares with the rows
      it received from the reduce-scatter.
    Returns the dict printed under "parity" (same on every rank)."""
    import torch
    import torch.distributed as dist

    n_loc = x1_l.shape[0]
    x1_all = torch.empty((N, x1_l.shape[1]), dtype=x1_l.dtype, device=dev)
    dist.all_gather_into_tensor(x1_all, x1_l.detach().contiguous())
    R = min(256, n_loc)
    e_hi = int(torch.searchsorted(rcv_l, torch.tensor([R], device=dev, dtype=rcv_l.dtype))[0])
    with torch.no_grad():
        ref = tp(x1_all, x2[:e_hi].detach(), w[:e_hi].detach(), indices_1=snd_l[:e_hi], indices_out=rcv_l[:e_hi], size_out=R)
    d_out = float((out[:R] - ref).abs().max())
    s_out = float(ref.abs().max())
    ok_out = d_out <= 1e-5 * s_out + 2e-6 * max(1.0, s_out)

    S = 32
    sel = torch.nonzero(snd_l < S).flatten()
    P = (S * 32 * 3) // world + 64
    cnt = torch.tensor([sel.numel()], device=dev, dtype=torch.int64)
    if sel.numel() > P:
        raise RuntimeError(f"parity check: {sel.numel()} edges from the sender window on rank {rank}, more than the {P} slots")

    def pad(t):
        buf = torch.zeros((P,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
        buf[: t.shape[0]] = t
        return buf

    parts = [pad(w[sel].detach()), pad(x2[sel].detach()), pad(cot[rcv_l[sel].long()]), pad(snd_l[sel])]
    gathered = []
    for t in parts + [cnt]:
        g = torch.empty((world,) + tuple(t.shape), dtype=t.dtype, device=dev)
        dist.all_gather_into_tensor(g, t.contiguous())
        gathered.append(g)
    d_g, s_g, ok_g = 0.0, 0.0, True
    if rank == 0:
        counts = gathered[4].flatten().tolist()
        w_g, x2_g, cot_g, snd_g = (torch.cat([g[r, : counts[r]] for r in range(world)]) for g in gathered[:4])
        win = x1_l[:S].detach().clone().requires_grad_(True)
        per_edge = tp(win, x2_g, w_g, indices_1=snd_g)
        (ref_g,) = torch.autograd.grad((per_edge * cot_g).sum(), win)
        d_g = float((gx1[:S] - ref_g).abs().max())
        s_g = float(ref_g.abs().max())
        ok_g = d_g <= 1e-4 * s_g + 2e-5 * max(1.0, s_g)
    flags = torch.tensor([float(ok_out), float(ok_g), d_out, d_g, s_g], device=dev, dtype=torch.float64)
    mins, maxs = flags.clone(), flags.clone()
    dist.all_reduce(mins, op=dist.ReduceOp.MIN)
    dist.all_reduce(maxs, op=dist.ReduceOp.MAX)
    return {"checked": "first 256 output rows of every rank vs the unsharded fused call; node-feature gradient rows of nodes 0..31 vs an unsharded evaluation of all edges that send from them",
            "out_rows_per_rank": R, "out_max_abs_diff": float(maxs[2]), "gx1_rows": S, "gx1_edges": int(sum(gathered[4].flatten().tolist())),
            "gx1_max_abs_diff": float(maxs[3]), "gx1_scale": float(maxs[4]), "ok": bool(mins[0] > 0 and mins[1] > 0)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--edges", type=int, default=E_TOTAL, help="total edges (default: the named configuration)")
    ap.add_argument("--nodes", type=int, default=N_TOTAL)
    ap.add_argument("--cpl", type=int, default=0, help="force channels per lane (2 or 4) in the channelwise kernels; 0 = library default")
    ap.add_argument("--exchange", default=None, choices=["peer_copy", "nccl"],
                    help="N>1: how node rows travel between ranks (default: copy engines over peer-mapped buffers)")
    ap.add_argument("--bundles", type=int, default=None, help="N>1: exchanges per direction (0 = one per irrep, 1, 2)")
    ap.add_argument("--nccl-ctas", type=int, default=0, help="N>1: upper bound on the thread blocks of a collective (0: NCCL's choice)")
    ap.add_argument("--sender-passes", type=int, default=None, help="backward: sender-range passes (1 = off)")
    ap.add_argument("--staging", type=int, default=None, help="forward staging: 0 = cp.async per lane, 1 = bulk copies")
    ap.add_argument("--bwd-variant", type=int, default=None, help="backward kernels: 1 = one warp per receiver, 2 = one thread block per receiver")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    import cuequivariance_b200 as cb
    from cuequivariance_b200 import profiling
    from cuequivariance_b200.dense import linear_f32x3
    from cuequivariance_b200.distributed import ReceiverShardedChannelWise, shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        from cuequivariance_b200.distributed import exchange_group_options

        dist.init_process_group("nccl", device_id=dev, pg_options=exchange_group_options(args.nccl_ctas))

    if args.cpl:
        from cuequivariance_b200 import channelwise

        channelwise.CHANNELS_PER_LANE = args.cpl
    if args.staging is not None:
        from cuequivariance_b200 import channelwise

        channelwise.STAGING = args.staging
    if args.bwd_variant is not None:
        from cuequivariance_b200 import channelwise

        channelwise.BWD_VARIANT = args.bwd_variant
    if args.exchange is not None:
        from cuequivariance_b200 import distributed

        distributed.EXCHANGE = args.exchange
    if args.bundles is not None:
        from cuequivariance_b200 import distributed

        distributed.BUNDLES = args.bundles
    if args.sender_passes is not None:
        from cuequivariance_b200 import channelwise

        channelwise.SENDER_PASSES = args.sender_passes
    E, N = args.edges, args.nodes
    tp = cb.ChannelWiseTensorProduct(IRREPS1, IRREPS2, FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    sh = cb.SphericalHarmonics([0, 1, 2, 3], normalize=True)
    mlp = make_mlp(tp.weight_numel, dev)

    # ---- synthetic graph (identical on every rank, then sharded) ---------------------------------
    gen = torch.Generator(device=dev).manual_seed(33)
    receivers = torch.sort(torch.randint(0, N, (E,), generator=gen, device=dev, dtype=torch.int32)).values
    senders = torch.randint(0, N, (E,), generator=gen, device=dev, dtype=torch.int32)
    n0, n1 = shard_bounds(N, world, rank)
    e0 = int(torch.searchsorted(receivers, torch.tensor([n0], device=dev, dtype=torch.int32))[0])
    e1 = int(torch.searchsorted(receivers, torch.tensor([n1], device=dev, dtype=torch.int32))[0])
    El = e1 - e0
    gen = torch.Generator(device=dev).manual_seed(30)
    x1_all = torch.randn(N, tp.irreps_in1.dim, generator=gen, device=dev)
    gen = torch.Generator(device=dev).manual_seed(31 + 1000 * rank)
    vec = torch.nn.functional.normalize(torch.randn(El, 3, generator=gen, device=dev), dim=1)
    length = 0.5 + 4.5 * torch.rand(El, generator=gen, device=dev)
    rcv_l = (receivers[e0:e1] - n0).contiguous()
    snd_l = senders[e0:e1].contiguous()
    x1_l = x1_all[n0:n1].contiguous()
    del x1_all, receivers, senders
    with torch.no_grad():
        x2 = sh(vec).contiguous()
        w = mlp(bessel(length)).contiguous()
    cot = torch.randn(n1 - n0, tp.irreps_out.dim, generator=gen, device=dev)
    # every step runs its backward before the next forward, so the backward may read the gathered node features
    # from the exchange's receive buffers instead of a copy
    op = ReceiverShardedChannelWise(tp, group=dist.group.WORLD if world > 1 else None, keep_gathered=False)

    def device_step():
        a, b, c = w.requires_grad_(True), x1_l.requires_grad_(True), x2.requires_grad_(True)
        out = op(b, c, a, snd_l, rcv_l)
        ga, gb, gc = torch.autograd.grad(out, (a, b, c), cot)
        return out, ga, gb, gc

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        device_step()
    barrier()
    profiling.reset()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        ev0.record()
        for _ in range(args.steps):
            device_step()
        ev1.record()
        barrier()
    launches = profiling.launch_count
    cb.check_status()   # raises if any bounded wait inside a kernel ran out during the timed steps
    ms = ev0.elapsed_time(ev1) / args.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    value = E / (ms * 1e-3)

    # ---- per-kernel durations (CUDA events around each native launch, on the launching stream) ----
    profiling.enable(True)
    profiling.reset()
    ksteps = 3
    for _ in range(ksteps):
        device_step()
    ksum = profiling.summary()
    profiling.enable(False)
    plan = tp.f._program(torch.float32)._special.plan
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = peaks.get("hbm_gbs", 6650.0)
    peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
    kernels = {}
    for g in plan.groups:
        for tag, bwd in (("cw_fwd", False), ("cw_bwd", True)):
            name = f"{tag}[{g['id']}]"
            if name in ksum:
                n, tot = ksum[name]
                bts = group_bytes(plan, g, El, n1 - n0, N, bwd)
                kernels[name] = {"ms": tot / n, "bytes": bts, "gbs": bts / (tot / n * 1e-3) / 1e9}
    dom = max(kernels, key=lambda k: kernels[k]["ms"]) if kernels else None
    total_kernel_ms = sum(v["ms"] for v in kernels.values())
    # algorithmic bytes of the step: every operand of the forward and of the backward call read or written
    # once (x2, both indices and the x2 gradient once per call, not once per group launch)
    w_sz, x1_sz, x2_sz, out_sz = plan.row_sizes
    n_loc = n1 - n0
    fwd_bytes = 4 * (El * (w_sz + x2_sz + 2) + N * x1_sz + n_loc * out_sz)
    bwd_bytes = fwd_bytes + 4 * (El * (w_sz + x2_sz) + N * x1_sz)
    total_bytes = fwd_bytes + bwd_bytes
    # measured DRAM bytes per edge of each launch come from one ncu capture (profiles/traffic.json); they are
    # only reported while the kernel sources are the ones that capture was taken on
    traffic, traffic_note = None, "no capture on record"
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))
        if rec.get("source_digest") != kernel_source_digest():
            traffic_note = "capture on record predates the current kernel sources"
        else:
            per_edge = rec["per_edge_bytes"].get(dom)
            traffic = per_edge * El if per_edge else None
            traffic_note = rec.get("source", "")
    except (OSError, ValueError, KeyError):
        pass
    # the same launch counted in float32 arithmetic: issued multiply-adds and multiplies per edge (from the ncu
    # capture on record) over the launch time, against the measured multiply-add peak of the CUDA cores
    fp32 = None
    try:
        per_edge = rec["fp32_instr_per_edge"].get(dom) if rec.get("source_digest") == kernel_source_digest() else None
        if per_edge:
            flop = 32.0 * (2.0 * per_edge["ffma"] + per_edge["fmul"]) * El
            tf = flop / (kernels[dom]["ms"] * 1e-3) / 1e12
            fp32 = {"achieved": tf, "peak": rec["fp32_peak_tflops"], "unit": "TFLOP/s", "frac": tf / rec["fp32_peak_tflops"],
                    "flop_per_edge": flop / El, "source": rec.get("fp32_source", ""), "peak_source": rec.get("fp32_peak_source", "")}
    except (NameError, KeyError, TypeError):
        pass
    roofline = None
    if dom:
        roofline = {"bound": "hbm", "kernel": dom, "achieved": kernels[dom]["gbs"], "peak": peak, "unit": "GB/s",
                    "frac": kernels[dom]["gbs"] / peak, "traffic": traffic, "traffic_note": traffic_note, "peak_source": peak_src, "fp32": fp32,
                    "all_kernels": {k: {"ms": round(v["ms"], 4), "gbs": round(v["gbs"], 1)} for k, v in kernels.items()},
                    "step_algorithmic_gbs": total_bytes / (total_kernel_ms * 1e-3) / 1e9 if total_kernel_ms else None,
                    "step_frac": (total_bytes / (ms * 1e-3) / 1e9) / peak}

    # ---- end to end: host buffers -> module API -> scalar on the host ------------------------------
    e2e = None
    if not args.no_e2e:
        h_x1 = x1_l.detach().cpu().pin_memory()
        h_vec = (vec * length[:, None]).cpu().pin_memory()
        h_snd, h_rcv = snd_l.cpu().pin_memory(), rcv_l.cpu().pin_memory()
        d_x1, d_vec = torch.empty_like(x1_l), torch.empty_like(vec)
        d_snd, d_rcv = torch.empty_like(snd_l), torch.empty_like(rcv_l)
        h_loss = torch.empty(1).pin_memory()
        params = list(mlp.parameters())

        copy_stream = torch.cuda.Stream(device=dev)
        x1_ready = torch.cuda.Event()

        def e2e_step():
            # the node features (the largest upload) travel on a copy stream while the radial MLP and the
            # spherical harmonics, which only need the edge vectors, already run
            main = torch.cuda.current_stream()
            copy_stream.wait_stream(main)
            d_vec.copy_(h_vec, non_blocking=True)      # small uploads first: the copy engine serves them in issue order
            d_snd.copy_(h_snd, non_blocking=True)
            d_rcv.copy_(h_rcv, non_blocking=True)
            with torch.cuda.stream(copy_stream):
                d_x1.copy_(h_x1, non_blocking=True)
                x1_ready.record(copy_stream)
            r = d_vec.norm(dim=1)
            hidden = mlp[1](mlp[0](bessel(r)))
            ww = linear_f32x3(hidden, mlp[2].weight, mlp[2].bias)   # the wide output layer on the tensor cores
            yy = sh(d_vec)
            main.wait_event(x1_ready)
            nodes = d_x1.detach().requires_grad_(True)
            out = op(nodes, yy, ww, d_snd, d_rcv)
            loss = (out * cot).sum()
            torch.autograd.grad(loss, [nodes] + params)
            h_loss.copy_(loss.detach().reshape(1), non_blocking=True)
            torch.cuda.current_stream().synchronize()

        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        ev0.record()
        for _ in range(args.steps):
            e2e_step()
        ev1.record()
        barrier()
        wall = (time.perf_counter() - t0) / args.steps * 1e3
        ems = max(ev0.elapsed_time(ev1) / args.steps, wall)
        t = torch.tensor([ems], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        h2d = h_x1.numel() * 4 + h_vec.numel() * 4 + h_snd.numel() * 4 + h_rcv.numel() * 4
        cb.check_status()
        e2e = {"value": E / (float(t[0]) * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
               "d2h": "scalar loss only (the output rows and the node-feature gradient stay on the device, as in a training step)",
               "ms_per_step": float(t[0]),
               "includes": "H2D of node features, edge vectors, indices; radial MLP (output layer: this library's 3xTF32 tcgen05 GEMM) and spherical harmonics on device; "
                           "TP fwd; backward to node features and MLP parameters; D2H of the scalar"}

    parity = None
    if world > 1:
        out, _, gx1, _ = device_step()
        parity = sharded_parity(tp, out.detach(), gx1, x1_l, x2, w, snd_l, rcv_l, cot, N, world, rank, dev)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        rate, cores, sec, kind = cpu_baseline()
        cpu = {"value": rate, "unit": "edges/s", "cores": cores, "kind": kind,
               "sample": f"{CPU_SAMPLE_EDGES} edges / {CPU_SAMPLE_NODES} nodes, same irreps and channels, fwd+bwd, {sec:.1f} s"}

    if rank == 0:
        print(json.dumps({
            "metric": "edges/s channelwise TP fwd+bwd (1M edges,128ch,lmax3)", "value": value, "unit": "edges/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"config 3: channelwise TP 128x(0e+1o+2e+3o) x (0e+1o+2e+3o) -> lmax 3, {E} edges, {N} nodes, "
                                   "mul_ir layout, sorted receivers, fwd+bwd (grads of weights, node features, harmonics)",
                       "sharding": f"edges by receiver range over {world} GPU(s); all-gather of node features, reduce-scatter of their gradient",
                       "l2": "inputs larger than L2 (per-edge weights alone are 12.3 GB); no explicit flush"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks.summary(),
            "parity": parity,
        }))
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit("sharded result differs from the single-GPU evaluation: " + json.dumps(parity))


if __name__ == "__main__":
    main()
