"""Throughput of the other benchmark configurations (the headline one is ``bench.py``).

    python bench_configs.py [--config 0|1|2|2bf16|4|linear|fma|fma2|all] [--steps K] [--batch B] [--edges E --nodes N]

``--batch`` scales configs 1, 2 and ``linear``, ``--edges`` / ``--nodes`` configs 0 and 4 (the profiles under
``profiles/`` are captured on scaled-down cases with these flags); ``fma`` / ``fma2`` measure the float32
multiply-add peak (scalar / packed instructions) that the CUDA-core kernels are rated against; ``linear`` is the
radial output layer of config 3 on its own (float32-accurate tensor-core GEMMs).

Prints one JSON line per configuration: device-timed (CUDA events) steps on seeded
synthetic inputs of the configuration's shapes, with the per-kernel breakdown of the native
launches.  Config 0: channelwise forward, 65,536 edges / 4,096 nodes / 128x(0e+1o+2e).
Config 1: symmetric contraction 128x(0e+1o+2e+3o) -> 128x(0e+1o), degree 3, 16,384 atoms, 10
species, forward + backward.  Config 2: fully connected 64x(0e+1o+2e)^3, batch 32,768, forward +
backward (float32: coupled operand in memory + three-pass TF32 GEMMs; ``2bf16``: fused kernels).  Config 4: config-3 graph at 65,536 edges, energy =
sum of the 0e outputs, first derivatives w.r.t. node features / harmonics / weights, then the
second derivative of their squared norm w.r.t. the same inputs (force-training pattern).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import cuequivariance_b200 as cb
from cuequivariance_b200 import profiling

FILTER = ["0e", "1o", "2e", "3o"]


def _time(step, steps, warmup=3):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    profiling.reset()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = profiling.launch_count // steps
    profiling.enable(True)
    profiling.reset()
    step()
    kernels = {k: round(v[1], 4) for k, v in profiling.summary().items()}
    profiling.enable(False)
    return ms, launches, kernels


def fma_peak(steps, dev, packed=False):
    """float32 FMA peak: 148 x 32 blocks of 256 threads, 16 independent chains each (`packed`: the same
    arithmetic issued as float32x2 instructions)."""
    import ctypes as C

    from cuequivariance_b200 import _lib

    sink = torch.zeros(1, device=dev)
    blocks, iters = 148 * 32, 20000
    entry = _lib.lib().cueq_b200_selftest_fma2_peak if packed else _lib.lib().cueq_b200_selftest_fma_peak
    fn = lambda: _lib.check(entry(C.c_void_p(sink.data_ptr()), blocks, iters,  # noqa: E731
                                  C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    for _ in range(3):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"config": "fma2" if packed else "fma",
            "what": "float32 multiply-add peak (register-resident chains" + (", packed float32x2 instructions)" if packed else ")"), "ms_per_step": ms,
            "tflops": 2.0 * blocks * 256 * 16 * iters / ms / 1e9}


def config0(steps, dev, E=65536, N=4096):
    tp = cb.ChannelWiseTensorProduct("128x0e+128x1o+128x2e", "0e+1o+2e+3o", FILTER, layout=cb.mul_ir,
                                     shared_weights=False, internal_weights=False)
    sh = cb.SphericalHarmonics([0, 1, 2, 3], normalize=True)
    g = torch.Generator(device=dev).manual_seed(0)
    x1 = torch.randn(N, tp.irreps_in1.dim, generator=g, device=dev)
    x2 = sh(torch.randn(E, 3, generator=g, device=dev))
    w = torch.randn(E, tp.weight_numel, generator=g, device=dev)
    snd = torch.randint(0, N, (E,), generator=g, device=dev, dtype=torch.int32)
    rcv = torch.randint(0, N, (E,), generator=g, device=dev, dtype=torch.int32)
    ms, n, k = _time(lambda: tp(x1, x2, w, indices_1=snd, indices_out=rcv, size_out=N), steps)
    return {"config": 0, "what": "channelwise forward, unsorted receivers", "ms_per_step": ms, "value": E / ms * 1e3, "unit": "edges/s",
            "gpu_launches": n, "kernels_ms": k}


def config1(steps, dev, B=16384):
    m = cb.SymmetricContraction("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o", 3, 10, layout=cb.mul_ir, dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev).manual_seed(10)
    x = torch.randn(B, m.irreps_in.dim, generator=g, device=dev, requires_grad=True)
    sp = torch.randint(0, 10, (B,), generator=g, device=dev)
    with torch.no_grad():
        m.weight.copy_(torch.randn(m.weight.shape, generator=g, device=dev) / 29 ** 0.5)

    def step():
        out = m(x, sp)
        torch.autograd.grad(out.sum(), [x, m.weight])

    ms, n, k = _time(step, steps)
    flops = (299_648 + 1_031_296) * B   # multiply-adds counted as 2 flop on the merged (unsymmetrised) polynomials, per atom
    return {"config": 1, "what": f"symmetric contraction fwd+bwd, {B} atoms", "ms_per_step": ms, "value": B / ms * 1e3, "unit": "atoms/s",
            "tflops": flops / ms / 1e9, "gpu_launches": n, "kernels_ms": k}


def config2(steps, dev, dtype=torch.float32, B=32768):
    s = "64x0e+64x1o+64x2e"
    m = cb.FullyConnectedTensorProduct(s, s, s, layout=cb.mul_ir, internal_weights=False, shared_weights=True)
    g = torch.Generator(device=dev).manual_seed(20)
    x1 = torch.randn(B, m.irreps_in1.dim, generator=g, device=dev).to(dtype).requires_grad_(True)
    x2 = torch.randn(B, m.irreps_in2.dim, generator=g, device=dev).to(dtype).requires_grad_(True)
    w = (torch.randn(1, m.weight_numel, generator=g, device=dev) / 64.0).to(dtype).requires_grad_(True)

    def step():
        out = m(x1, x2, w)
        torch.autograd.grad(out.float().sum(), [x1, x2, w])

    ms, n, k = _time(step, steps)
    route = "fused tcgen05 kernels (coupled operand built on chip, bf16 operands, float32 accumulation)" if dtype == torch.bfloat16 \
        else "float32-accurate route (coupled operand in memory, three-pass TF32 tcgen05 GEMMs)"
    flops = 4 * 2 * 35 * 64 ** 3 * B
    peak = _peaks().get("bf16_tflops_sustained")
    return {"config": 2, "what": f"fully connected fwd+bwd, {str(dtype).split('.')[-1]}, {B} samples, {route}", "ms_per_step": ms,
            "value": B / ms * 1e3, "unit": "samples/s", "tflops": flops / ms / 1e9,
            "roofline": {"bound": "tensor", "achieved": flops / ms / 1e9, "peak": peak, "unit": "TFLOP/s",
                         "frac": (flops / ms / 1e9) / peak if peak else None,
                         "note": "useful flop of the four contractions over the measured sustained bf16 peak; the float32 route spends three TF32 passes per product"},
            "gpu_launches": n, "kernels_ms": k}


def dense_layer(steps, dev, rows=1048576):
    """The radial output layer of config 3 on its own: ``linear_f32x3`` rows x 64 -> 2,944 forward + backward."""
    from cuequivariance_b200.dense import linear_f32x3

    g = torch.Generator(device=dev).manual_seed(50)
    x = torch.randn(rows, 64, generator=g, device=dev, requires_grad=True)
    w = (torch.randn(2944, 64, generator=g, device=dev) / 8.0).requires_grad_(True)
    b = torch.zeros(2944, device=dev, requires_grad=True)
    cot = torch.randn(rows, 2944, generator=g, device=dev)

    def step():
        torch.autograd.grad(linear_f32x3(x, w, b), [x, w, b], cot)

    ms, n, k = _time(step, steps)
    flops = 3 * 2 * rows * 64 * 2944
    return {"config": "linear", "what": f"float32-accurate dense layer {rows} x 64 -> 2944, fwd+bwd", "ms_per_step": ms,
            "tflops": flops / ms / 1e9, "gpu_launches": n, "kernels_ms": k}


def _peaks():
    try:
        return json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")))
    except OSError:
        return {}


def config4(steps, dev, E=65536, N=4096):
    s1 = "+".join(f"128x{ir}" for ir in FILTER)
    tp = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    sh = cb.SphericalHarmonics([0, 1, 2, 3], normalize=True)
    g = torch.Generator(device=dev).manual_seed(40)
    x1 = torch.randn(N, tp.irreps_in1.dim, generator=g, device=dev, requires_grad=True)
    vec = torch.randn(E, 3, generator=g, device=dev, requires_grad=True)
    w = torch.randn(E, tp.weight_numel, generator=g, device=dev, requires_grad=True)
    snd = torch.randint(0, N, (E,), generator=g, device=dev, dtype=torch.int32)
    rcv = torch.sort(torch.randint(0, N, (E,), generator=g, device=dev, dtype=torch.int32)).values

    def step():
        out = tp(x1, sh(vec), w, indices_1=snd, indices_out=rcv, size_out=N)
        energy = out[:, :512].sum()
        gx, gv, gw = torch.autograd.grad(energy, (x1, vec, w), create_graph=True)
        loss = gv.pow(2).sum()
        torch.autograd.grad(loss, (x1, vec, w), allow_unused=True)

    ms, n, k = _time(step, steps)
    return {"config": 4, "what": f"energy -> forces -> force loss gradient (double backward), {E} edges", "ms_per_step": ms,
            "value": E / ms * 1e3, "unit": "edges/s", "gpu_launches": n, "kernels_ms": k}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="all")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--edges", type=int, default=65536, help="configs 0 and 4: number of edges")
    ap.add_argument("--nodes", type=int, default=4096, help="configs 0 and 4: number of nodes")
    ap.add_argument("--batch", type=int, default=None, help="configs 1 and 2: atoms / samples (default: the configuration's size)")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    fns = {"0": lambda steps, dev: config0(steps, dev, a.edges, a.nodes),
           "1": lambda steps, dev: config1(steps, dev, a.batch or 16384),
           "2": lambda steps, dev: config2(steps, dev, torch.float32, a.batch or 32768),
           "2bf16": lambda steps, dev: config2(steps, dev, torch.bfloat16, a.batch or 32768),
           "4": lambda steps, dev: config4(steps, dev, a.edges, a.nodes),
           "linear": lambda steps, dev: dense_layer(steps, dev, a.batch or 1048576),
           "fma": fma_peak, "fma2": lambda steps, dev: fma_peak(steps, dev, packed=True)}
    for key in ([k for k in fns if not k.startswith("fma") and k != "linear"] if a.config == "all" else [a.config]):
        print(json.dumps(fns[key](a.steps, dev)), flush=True)


if __name__ == "__main__":
    main()
