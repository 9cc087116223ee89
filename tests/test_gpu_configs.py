"""GPU parity of the benchmark configurations, at their stated sizes, against the CPU oracle.

* config 0 at full size (65,536 edges, 4,096 nodes, 128x(0e+1o+2e), unsorted int32 indices):
  the whole output against the oracle streamed over edge chunks, float32 and float64 oracles;
* config 3 at full size (1,048,576 edges, 32,768 nodes, radial-MLP weights, sorted receivers):
  forward and backward run on the full graph; the oracle checks them on a fixed sub-graph -
  the output rows, weight gradient and harmonics gradient of a window of receivers (all of
  their edges), and the node-feature gradient rows of a window of senders (all of *their*
  edges, wherever the receivers are);
* config 4 (force-training chain) at 65,536 edges / 4,096 nodes: edge vectors -> spherical
  harmonics and -> lengths -> Bessel -> MLP -> weights; energy = sum of the 0e outputs; first
  derivatives; then the gradient of the squared norm of the derivative w.r.t. the edge vectors
  ("forces") w.r.t. edge vectors, node features and MLP parameters.  float64 within 1e-12 of
  the float64 oracle, float32 within the float32 tolerance of both oracles;
* config 1 (symmetric contraction, 128 channels, degree 3, 10 species) on a 512-atom slice,
  forward and backward, with the straight-line kernels asserted to have run;
* config 2 (fully connected, 64 channels) on a 192-sample slice, bf16 and float32, forward and
  backward, with each route's kernels asserted.

Every float32 comparison also records by how much the stated tolerance (1e-5 relative, 1e-6
absolute) is exceeded against each oracle (`tests/_tolerance.py`).
"""
import math

import pytest
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import descriptors as D, profiling
from cuequivariance_b200.stp import SegmentedTensorProduct
from cuequivariance_b200.polynomial import Polynomial
from oracle import chunked, naive

from _tolerance import close, report

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FILTER = ["0e", "1o", "2e", "3o"]
IR3 = "+".join(f"128x{ir}" for ir in FILTER)


def _sh_cpu(vec):
    e = D.spherical_harmonics("1o", [0, 1, 2, 3])
    return naive.segmented_polynomial(e.polynomial, [torch.nn.functional.normalize(vec, dim=1)])[0]


def _bessel(r, n=8, rc=5.0):
    k = torch.arange(1, n + 1, device=r.device, dtype=r.dtype) * math.pi / rc
    return math.sqrt(2.0 / rc) * torch.sin(k * r[:, None]) / r[:, None]


def _blocks(e):
    return [(m, ir.dim) for m, ir in e.inputs[1].irreps], [(m, ir.dim) for m, ir in e.outputs[0].irreps]


# ---- config 0 ------------------------------------------------------------------------------------
def test_config0_full_size_matches_oracle():
    s1 = "128x0e+128x1o+128x2e"
    E, N = 65536, 4096
    e = D.channelwise_tensor_product(s1, "0e+1o+2e+3o", FILTER)
    b1, bo = _blocks(e)
    tp = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    x1 = torch.randn(N, tp.irreps_in1.dim, generator=torch.Generator().manual_seed(0), dtype=torch.float64)
    x2 = _sh_cpu(torch.randn(E, 3, generator=torch.Generator().manual_seed(1), dtype=torch.float64))
    w = torch.randn(E, tp.weight_numel, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    g = torch.Generator().manual_seed(3)
    snd, rcv = torch.randint(0, N, (E,), generator=g), torch.randint(0, N, (E,), generator=g)
    profiling.reset()
    got = tp(x1.float().to(DEV), x2.float().to(DEV), w.float().to(DEV), indices_1=snd.int().to(DEV), indices_out=rcv.int().to(DEV), size_out=N)
    assert profiling.launch_count == 3, "the specialised channelwise kernels did not run"
    refs = {}
    for name, dt in (("f32", torch.float32), ("f64", torch.float64)):
        xs = [w.to(dt), naive.transpose_layout(x1.to(dt), b1, True), x2.to(dt)]
        (o,) = chunked.forward(e.polynomial, xs, {1: snd}, {0: N}, {0: rcv}, E, chunk=8192, accumulate_dtype=dt)
        refs[name] = naive.transpose_layout(o, bo, False)
    report("0 (65,536 edges, full size)", "out", got, refs["f32"], refs["f64"])
    close(got, refs["f64"], 1e-5, 2e-6, "out vs float64 oracle")
    close(got, refs["f32"], 1e-5, 2e-6, "out vs float32 oracle")


# ---- config 3 ------------------------------------------------------------------------------------
def test_config3_full_size_matches_oracle_on_a_subgraph():
    E, N = 1_048_576, 32_768
    e = D.channelwise_tensor_product(IR3, "0e+1o+2e+3o", FILTER)
    b1, bo = _blocks(e)
    tp = cb.ChannelWiseTensorProduct(IR3, "0e+1o+2e+3o", FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    sh = cb.SphericalHarmonics([0, 1, 2, 3], normalize=True)
    gd = lambda s: torch.Generator(device=DEV).manual_seed(s)  # noqa: E731
    x1 = torch.randn(N, tp.irreps_in1.dim, generator=gd(30), device=DEV)
    g31 = gd(31)
    unit = torch.nn.functional.normalize(torch.randn(E, 3, generator=g31, device=DEV), dim=1)
    length = 0.5 + 4.5 * torch.rand(E, generator=g31, device=DEV)
    torch.manual_seed(32)
    mlp = torch.nn.Sequential(torch.nn.Linear(8, 64), torch.nn.SiLU(), torch.nn.Linear(64, tp.weight_numel)).to(DEV)
    g33 = gd(33)
    rcv = torch.sort(torch.randint(0, N, (E,), generator=g33, device=DEV, dtype=torch.int32)).values
    snd = torch.randint(0, N, (E,), generator=g33, device=DEV, dtype=torch.int32)
    with torch.no_grad():
        x2 = sh(unit).contiguous()
        w = mlp(_bessel(length)).contiguous()
    cot = torch.randn(N, tp.irreps_out.dim, generator=gd(34), device=DEV)
    a, b, c = w.requires_grad_(True), x1.requires_grad_(True), x2.requires_grad_(True)
    profiling.reset()
    out = tp(b, c, a, indices_1=snd, indices_out=rcv, size_out=N)
    gw, gx1, gx2 = torch.autograd.grad(out, (a, b, c), cot)
    assert profiling.launch_count == 8, "the specialised channelwise kernels did not run"

    # receiver window: all edges of receivers [r0, r0 + R)
    r0, R = 20_000, 256
    e0 = int(torch.searchsorted(rcv, torch.tensor([r0], device=DEV, dtype=torch.int32))[0])
    e1 = int(torch.searchsorted(rcv, torch.tensor([r0 + R], device=DEV, dtype=torch.int32))[0])
    assert 6000 < e1 - e0 < 11000
    w_s, x2_s = w[e0:e1].detach().cpu(), x2[e0:e1].detach().cpu()
    snd_s, rcv_s = snd[e0:e1].long().cpu(), (rcv[e0:e1].long() - r0).cpu()
    x1_c, cot_r = x1.detach().cpu(), cot[r0 : r0 + R].cpu()
    res = {}
    for name, dt in (("f32", torch.float32), ("f64", torch.float64)):
        cot_dt = cot_r.to(dt)
        outs = []

        def fn(rows, whole, dt=dt, cot_dt=cot_dt, outs=outs):
            w_, x2_, s_, r_ = rows
            (o,) = naive.segmented_polynomial(e.polynomial, [w_, naive.transpose_layout(whole[0], b1, True), x2_], {1: s_}, {0: R}, {0: r_})
            o = naive.transpose_layout(o, bo, False)
            outs.append(o.detach())
            return (o * cot_dt).sum()

        _, g_rows, _ = chunked.value_and_grads(fn, [w_s.to(dt), x2_s.to(dt), snd_s, rcv_s], [x1_c.to(dt)], e1 - e0, chunk=2048, accumulate_dtype=dt)
        res[name] = (sum(outs[1:], outs[0]), g_rows[0], g_rows[1])
    for k, (name, got) in enumerate((("out", out[r0 : r0 + R]), ("grad w", gw[e0:e1]), ("grad x2", gx2[e0:e1]))):
        report("3 (1,048,576 edges; receiver window)", name, got, res["f32"][k], res["f64"][k])
        m = 1 if k == 0 else 10
        close(got, res["f64"][k], m * 1e-5, m * 2e-6, name + " vs float64 oracle")
        close(got, res["f32"][k], m * 1e-5, m * 2e-6, name + " vs float32 oracle")

    # sender window: the gradient rows of nodes [s0, s0 + S) collect edges from all over the graph
    s0, S = 5_000, 256
    mask = (snd >= s0) & (snd < s0 + S)
    idx = torch.nonzero(mask).flatten()
    n_e = idx.numel()
    assert 6000 < n_e < 11000
    w_s, x2_s = w[idx].detach().cpu(), x2[idx].detach().cpu()
    snd_s = (snd[idx].long() - s0).cpu()
    cot_e = cot[rcv[idx].long()].cpu()     # cotangent row of each edge's receiver
    x1_w = x1[s0 : s0 + S].detach().cpu()
    gx1_ref = {}
    for name, dt in (("f32", torch.float32), ("f64", torch.float64)):
        def fn(rows, whole, dt=dt):
            w_, x2_, s_, c_ = rows
            (o,) = naive.segmented_polynomial(e.polynomial, [w_, naive.transpose_layout(whole[0], b1, True), x2_], {1: s_})
            return (naive.transpose_layout(o, bo, False) * c_.detach()).sum()

        _, _, g_whole = chunked.value_and_grads(fn, [w_s.to(dt), x2_s.to(dt), snd_s, cot_e.to(dt)], [x1_w.to(dt)], n_e, chunk=2048, accumulate_dtype=dt)
        gx1_ref[name] = g_whole[0]
    report("3 (1,048,576 edges; sender window)", "grad x1", gx1[s0 : s0 + S], gx1_ref["f32"], gx1_ref["f64"])
    close(gx1[s0 : s0 + S], gx1_ref["f64"], 1e-4, 2e-5, "grad x1 vs float64 oracle")
    close(gx1[s0 : s0 + S], gx1_ref["f32"], 1e-4, 2e-5, "grad x1 vs float32 oracle")


# ---- config 4 ------------------------------------------------------------------------------------
def _energy_polynomial(e):
    """The channelwise polynomial restricted to the paths that feed the 0e output blocks (the
    energy is the sum of those blocks, so no other path contributes to it or its derivatives)."""
    ope, d = e.polynomial.operations[0]
    scalar_segments = {s for s, seg in enumerate(d.operands[3].segments) if seg[0] == 1}
    keep = [p for p in d.paths if p.indices[3] in scalar_segments]
    assert len(keep) == 4
    d0 = SegmentedTensorProduct(d.operand_subscripts, d.coefficient_subscripts, list(d.operands), keep)
    return Polynomial(e.polynomial.inputs, e.polynomial.outputs, [(ope, d0)])


def _chain_inputs(E, N, dtype):
    g = torch.Generator().manual_seed(40)
    x1 = torch.randn(N, 2048, generator=g, dtype=torch.float64)
    unit = torch.nn.functional.normalize(torch.randn(E, 3, generator=g, dtype=torch.float64), dim=1)
    vec = unit * (0.5 + 4.5 * torch.rand(E, 1, generator=g, dtype=torch.float64))
    snd = torch.randint(0, N, (E,), generator=g)
    rcv = torch.sort(torch.randint(0, N, (E,), generator=g)).values
    torch.manual_seed(41)
    mlp = torch.nn.Sequential(torch.nn.Linear(8, 64), torch.nn.SiLU(), torch.nn.Linear(64, 2944)).double()
    params = [p.detach().clone() for p in mlp.parameters()]   # W1, b1, W2, b2
    return [t.to(dtype) for t in (x1, vec)], snd, rcv, [p.to(dtype) for p in params]


def _weights(vec, params):
    W1, c1, W2, c2 = params
    h = torch.nn.functional.silu(_bessel(vec.norm(dim=1)) @ W1.t() + c1)
    return h @ W2.t() + c2


NAMES4 = ["energy", "dE/dx1", "dE/dx2", "dE/dw", "dE/dvec", "dS/dvec", "dS/dx1", "dS/dW1", "dS/db1", "dS/dW2", "dS/db2"]


def _chain_cuda(tp, sh, x1, vec, snd, rcv, params, N):
    x1, vec = x1.to(DEV).requires_grad_(True), vec.to(DEV).requires_grad_(True)
    params = [p.to(DEV).requires_grad_(True) for p in params]
    x2 = sh(vec)
    w = _weights(vec, params)
    out = tp(x1, x2, w, indices_1=snd.int().to(DEV), indices_out=rcv.int().to(DEV), size_out=N)
    energy = out[:, :512].sum()
    g_x1, g_x2, g_w, g_vec = torch.autograd.grad(energy, (x1, x2, w, vec), create_graph=True)
    S = g_vec.pow(2).sum()
    second = torch.autograd.grad(S, [vec, x1] + params)
    return [energy.detach(), g_x1.detach(), g_x2.detach(), g_w.detach(), g_vec.detach()] + [t.detach() for t in second]


def _chain_oracle(e, x1, vec, snd, rcv, params, N, chunk=8192):
    p0 = _energy_polynomial(e)
    b1, _ = _blocks(e)
    sh_poly = D.spherical_harmonics("1o", [0, 1, 2, 3]).polynomial
    dt = x1.dtype
    E = vec.shape[0]
    energy = torch.zeros((), dtype=dt)
    g_x1 = torch.zeros_like(x1)

    def pieces(rows, whole):
        v, s_, r_ = rows
        x1_, *pr = whole
        x2 = naive.segmented_polynomial(sh_poly, [torch.nn.functional.normalize(v, dim=1)])[0]
        w = _weights(v, pr)
        (o,) = naive.segmented_polynomial(p0, [w, naive.transpose_layout(x1_, b1, True), x2], {1: s_}, {0: N}, {0: r_})
        en = o.sum()
        gx1, gx2, gw, gv = torch.autograd.grad(en, (x1_, x2, w, v), create_graph=True)
        return en, gx1, gx2, gw, gv

    def fn(rows, whole):
        nonlocal energy, g_x1
        en, gx1, _, _, gv = pieces(rows, whole)
        energy = energy + en.detach()
        g_x1 = g_x1 + gx1.detach()
        return gv.pow(2).sum()

    def extra(rows, whole):
        _, _, gx2, gw, gv = pieces(rows, whole)
        return [gx2, gw, gv]

    _, g_rows, g_whole, first = chunked.value_and_grads(fn, [vec, snd, rcv], [x1] + list(params), E, chunk=chunk, accumulate_dtype=dt, extra=extra)
    return [energy, g_x1, first[0], first[1], first[2], g_rows[0], g_whole[0]] + g_whole[1:]


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_config4_force_training_chain_matches_oracle(tag):
    E, N = 65536, 4096
    e = D.channelwise_tensor_product(IR3, "0e+1o+2e+3o", FILTER)
    tp = cb.ChannelWiseTensorProduct(IR3, "0e+1o+2e+3o", FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    sh = cb.SphericalHarmonics([0, 1, 2, 3], normalize=True)
    dtype = torch.float64 if tag == "f64" else torch.float32
    (x1, vec), snd, rcv, params = _chain_inputs(E, N, dtype)
    profiling.reset()
    got = _chain_cuda(tp, sh, x1, vec, snd, rcv, params, N)
    assert profiling.launch_count > 0
    (x1d, vecd), _, _, paramsd = _chain_inputs(E, N, torch.float64)
    if tag == "f32":   # the float64 oracle sees the float32-rounded inputs
        x1d, vecd, paramsd = x1.double(), vec.double(), [p.double() for p in params]
    ref64 = _chain_oracle(e, x1d, vecd, snd, rcv, paramsd, N)
    if tag == "f64":
        for name, a, b in zip(NAMES4, got, ref64):
            close(a, b, 1e-12, 1e-12, name)
        return
    ref32 = _chain_oracle(e, x1, vec, snd, rcv, params, N)
    for k, (name, a, b32, b64) in enumerate(zip(NAMES4, got, ref32, ref64)):
        report("4 (65,536 edges, chain to edge vectors)", name, a, b32, b64)
        m = 1 if k == 0 else (10 if k < 5 else 100)
        close(a, b64, m * 1e-5, m * 2e-6, name + " vs float64 oracle")
        close(a, b32, m * 1e-5, m * 2e-6, name + " vs float32 oracle")


# ---- config 1 ------------------------------------------------------------------------------------
def test_config1_128_channels_matches_oracle():
    B = 512
    m = cb.SymmetricContraction("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o", 3, 10, layout=cb.mul_ir, dtype=torch.float32, device=DEV)
    e = m.etp
    bi = [(mu, ir.dim) for mu, ir in e.inputs[1].irreps]
    bo = [(mu, ir.dim) for mu, ir in e.outputs[0].irreps]
    x = torch.randn(B, m.irreps_in.dim, generator=torch.Generator().manual_seed(10), dtype=torch.float64)
    sp = torch.randint(0, 10, (B,), generator=torch.Generator().manual_seed(11))
    wt = torch.randn(10, *m.weight_shape, generator=torch.Generator().manual_seed(12), dtype=torch.float64) / math.sqrt(m.weight_shape[0])
    cot = torch.randn(B, m.irreps_out.dim, generator=torch.Generator().manual_seed(13), dtype=torch.float64)

    def run(fn, xs, c):
        xs = [t.clone().requires_grad_(True) for t in xs]
        o = fn(*xs)
        return [o.detach()] + list(torch.autograd.grad((o * c).sum(), xs))

    def ref_fn(w_, x_):
        (o,) = naive.segmented_polynomial(e.polynomial, [w_.flatten(1), naive.transpose_layout(x_, bi, True)], {0: sp})
        return naive.transpose_layout(o, bo, False)

    def got_fn(w_, x_):
        out = m.f([w_.flatten(1), m.transpose_in(x_)], input_indices={0: sp.to(DEV)})
        return m.transpose_out(out[0])

    profiling.reset()
    profiling.enable()
    try:
        got = run(got_fn, [wt.float().to(DEV), x.float().to(DEV)], cot.float().to(DEV))
        names = set(profiling.summary())
    finally:
        profiling.enable(False)
    assert any(n.startswith("u1d_static") for n in names) and not any(n.startswith("u1d_generic") for n in names), names
    ref32 = run(ref_fn, [wt.float(), x.float()], cot.float())
    ref64 = run(ref_fn, [wt, x], cot)
    for k, (name, a, b32, b64) in enumerate(zip(["out", "grad weight", "grad x"], got, ref32, ref64)):
        report("1 (128 channels, 512 atoms)", name, a, b32, b64)
        f = 1 if k == 0 else 10
        close(a, b64, f * 1e-5, f * 2e-6, name + " vs float64 oracle")
        close(a, b32, f * 1e-5, f * 2e-6, name + " vs float32 oracle")


# ---- config 2 ------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["bf16", "f32"])
def test_config2_64_channels_matches_oracle(tag):
    s = "64x0e+64x1o+64x2e"
    B = 192
    e = D.fully_connected_tensor_product(s, s, s)
    m = cb.FullyConnectedTensorProduct(s, s, s, layout=cb.ir_mul, internal_weights=False, shared_weights=True)
    dt = torch.bfloat16 if tag == "bf16" else torch.float32
    x1 = torch.randn(B, m.irreps_in1.dim, generator=torch.Generator().manual_seed(20), dtype=torch.float64).to(dt)
    x2 = torch.randn(B, m.irreps_in2.dim, generator=torch.Generator().manual_seed(21), dtype=torch.float64).to(dt)
    w = (torch.randn(1, m.weight_numel, generator=torch.Generator().manual_seed(22), dtype=torch.float64) / 64.0).to(dt)
    cot = torch.randn(B, m.irreps_out.dim, generator=torch.Generator().manual_seed(23), dtype=torch.float64)

    def run(fn, xs, c):
        xs = [t.clone().requires_grad_(True) for t in xs]
        o = fn(*xs)
        return [o.detach()] + list(torch.autograd.grad((o.to(c.dtype) * c).sum(), xs))

    ref_fn = lambda w_, a, b: naive.segmented_polynomial(e.polynomial, [w_, a, b])[0]  # noqa: E731
    profiling.reset()
    profiling.enable()
    try:
        got = run(lambda w_, a, b: m(a, b, w_), [w.to(DEV), x1.to(DEV), x2.to(DEV)], cot.float().to(DEV))
        names = set(profiling.summary())
    finally:
        profiling.enable(False)
    ref64 = run(ref_fn, [w.double(), x1.double(), x2.double()], cot)
    if tag == "bf16":
        assert {"fctp_fused_forward", "fctp_fused_gw", "fctp_fused_gx1", "fctp_fused_gx2"} <= names, names
        for name, a, b in zip(["out", "grad w", "grad x1", "grad x2"], got, ref64):
            scale = float(b.abs().max())
            err = float((a.double().cpu() - b).abs().max())
            assert err <= 2e-2 * scale, f"{name}: max abs diff {err:.3e} at scale {scale:.3e}"
        return
    assert {"fctp_f32_forward", "fctp_f32_gw", "fctp_f32_gx"} <= names, names
    ref32 = run(ref_fn, [w, x1, x2], cot.float())
    for k, (name, a, b32, b64) in enumerate(zip(["out", "grad w", "grad x1", "grad x2"], got, ref32, ref64)):
        report("2 float32 (64 channels, 192 samples)", name, a, b32, b64)
        f = 1 if k == 0 else 10
        close(a, b64, f * 1e-5, f * 2e-6, name + " vs float64 oracle")
        close(a, b32, f * 1e-5, f * 2e-6, name + " vs float32 oracle")
