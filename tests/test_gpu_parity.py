"""GPU parity tests: the CUDA executor (called through the C-ABI library) against the
reference-generated golden fixtures and against the CPU oracle on seeded inputs.

Tolerances: float64 1e-12 relative+absolute; float32 1e-5 relative / 2e-6 absolute on
outputs (x10 for first derivatives, x100 for the second-order check, following the
reference tests' scaling, cuequivariance_torch/tests/primitives/segmented_polynomial_test.py:174-175).
"""
import itertools

import numpy as np
import pytest
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import descriptors as D, profiling
from oracle import naive

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"f64": (1e-12, 1e-12), "f32": (1e-5, 2e-6)}
DT = {"f64": torch.float64, "f32": torch.float32}


def _t(a, device=DEV):
    return torch.from_numpy(np.array(a)).to(device)


def _derivatives(fn, inputs, cot):
    xs = [x.clone().requires_grad_(True) for x in inputs]
    out = fn(*xs)
    g1 = torch.autograd.grad((out * cot).sum(), xs, retain_graph=True, allow_unused=True)
    gg = torch.autograd.grad(out.pow(2).sum(), xs, create_graph=True, allow_unused=True)
    tot = sum(g.pow(2).sum() for g in gg if g is not None)
    g2 = torch.autograd.grad(tot, xs, allow_unused=True)
    return out.detach(), g1, g2


def _close(a, b, rtol, atol, what=""):
    a = a.detach().cpu().double().numpy() if torch.is_tensor(a) else np.asarray(a, dtype=np.float64)
    b = b.detach().cpu().double().numpy() if torch.is_tensor(b) else np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    scale = max(1.0, float(np.abs(b).max())) if b.size else 1.0  # absolute term in units of the tensor's magnitude
    err = np.abs(a - b) - (atol * scale + rtol * np.abs(b))
    assert np.all(err <= 0), f"{what}: max abs diff {np.abs(a - b).max():.3e}, worst excess {err.max():.3e}"


def _check_golden(g, out, g1, g2, rtol, atol):
    _close(out, g["out"], rtol, atol, "out")
    for i, (a, b) in enumerate(zip(g1, g2)):
        _close(a, g[f"grad{i}"], 10 * rtol, 10 * atol, f"grad{i}")
        _close(b, g[f"gradgrad{i}"], 100 * rtol, 100 * atol, f"gradgrad{i}")


@pytest.mark.parametrize("tag", ["f64", "f32"])
@pytest.mark.parametrize("name,s1", [("cw_l2", "8x0e+8x1o+8x2e"), ("cw_l3", "8x0e+8x1o+8x2e+8x3o")])
def test_channelwise_module_golden(golden, name, s1, tag):
    g = golden(f"{name}_module_{tag}.npz")
    m = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", ["0e", "1o", "2e", "3o"], layout=cb.mul_ir,
                                    shared_weights=False, internal_weights=False)
    N = g["x1"].shape[0]
    for idx_dtype in (torch.int64, torch.int32):
        snd, rcv = _t(g["senders"]).to(idx_dtype), _t(g["receivers"]).to(idx_dtype)
        out, g1, g2 = _derivatives(
            lambda w, a, b: m(a, b, w, indices_1=snd, indices_out=rcv, size_out=N),
            [_t(g["w"]), _t(g["x1"]), _t(g["x2"])], _t(g["cot"]))
        _check_golden(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_uniform1d_index_modes_golden(golden, tag):
    e = D.channelwise_tensor_product("16x0e+16x1o", "0e+1o+2e", "0e+1o")
    f = cb.SegmentedPolynomial(e.polynomial, method="uniform_1d")
    g = golden(f"u1d_indexed_{tag}.npz")
    ia, io = _t(g["ia"]), _t(g["io"])
    out, g1, g2 = _derivatives(
        lambda a, b, c: f([a, b, c], {0: ia}, {0: torch.empty(3, 1, device=DEV)}, {0: io})[0],
        [_t(g["a"]), _t(g["b"]), _t(g["c"])], _t(g["cot"]))
    _check_golden(g, out, g1, g2, *TOL[tag])
    g = golden(f"u1d_sum_{tag}.npz")
    a = _t(g["a"])
    out, g1, g2 = _derivatives(
        lambda b, c: f([a, b, c], {}, {0: torch.empty(1, 1, device=DEV)}, {})[0], [_t(g["b"]), _t(g["c"])], _t(g["cot"]))
    _check_golden(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_symmetric_contraction_module_golden(golden, tag):
    g = golden(f"symmetric_contraction_module_{tag}.npz")
    m = cb.SymmetricContraction("4x0e+4x1o+4x2e+4x3o", "4x0e+4x1o", 3, 10, layout=cb.mul_ir, dtype=DT[tag], device=DEV)
    sp = _t(g["species"])

    def fn(w, x):
        out = m.f([w.flatten(1), m.transpose_in(x)], input_indices={0: sp})
        return m.transpose_out(out[0])

    out, g1, g2 = _derivatives(fn, [_t(g["weight"]), _t(g["x"])], _t(g["cot"]))
    _check_golden(g, out, g1, g2, *TOL[tag])
    # and through the module's own forward with its parameter
    with torch.no_grad():
        m.weight.copy_(_t(g["weight"]))
    _close(m(_t(g["x"]), sp.to(torch.int32)), g["out"], *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_fully_connected_module_golden(golden, tag):
    g = golden(f"fully_connected_module_{tag}.npz")
    s = "4x0e+4x1o+4x2e"
    m = cb.FullyConnectedTensorProduct(s, s, s, layout=cb.mul_ir, internal_weights=False, shared_weights=True)
    out, g1, g2 = _derivatives(lambda w, a, b: m(a, b, w), [_t(g["weight"]), _t(g["x1"]), _t(g["x2"])], _t(g["cot"]))
    _check_golden(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_spherical_harmonics_golden(golden, tag):
    g = golden(f"spherical_harmonics_{tag}.npz")
    sh = cb.SphericalHarmonics([0, 1, 2, 3], normalize=True)
    out, g1, g2 = _derivatives(lambda v: sh(v), [_t(g["vec"])], _t(g["cot"]))
    _check_golden(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_transpose_golden(golden, tag):
    g = golden(f"transpose_{tag}.npz")
    t = cb.TransposeIrrepsLayout("3x0e+5x1o+2x2e", source=cb.mul_ir, target=cb.ir_mul)
    x = _t(g["x"]).requires_grad_(True)
    y = t(x)
    assert np.array_equal(y.detach().cpu().numpy(), g["y"])
    back = cb.TransposeIrrepsLayout("3x0e+5x1o+2x2e", source=cb.ir_mul, target=cb.mul_ir)
    assert torch.equal(back(y), x)
    (gx,) = torch.autograd.grad((y * y).sum(), x)
    assert torch.equal(gx, 2 * x.detach())


# ---- every shared / batched / indexed combination against the oracle (the matrix of the
# ---- reference's executor tests, segmented_polynomial_test.py:286-301) ------------------
MODES = ["shared", "batched", "indexed"]


def _make_operand(mode, size, batch, rows, gen, dtype):
    if mode == "shared":
        return torch.randn(1, size, generator=gen, dtype=torch.float64).to(dtype), None
    if mode == "batched":
        return torch.randn(batch, size, generator=gen, dtype=torch.float64).to(dtype), None
    idx = torch.sort(torch.randint(0, rows, (batch,), generator=gen)).values
    return torch.randn(rows, size, generator=gen, dtype=torch.float64).to(dtype), idx


@pytest.mark.parametrize("tag", ["f64", "f32"])
@pytest.mark.parametrize("out_mode", MODES)
@pytest.mark.parametrize("in_modes", list(itertools.product(MODES, repeat=3)))
def test_index_mode_matrix_against_oracle(in_modes, out_mode, tag):
    if all(m == "shared" for m in in_modes) and out_mode == "batched":
        pytest.skip("no batch axis anywhere")
    dtype = DT[tag]
    e = D.channelwise_tensor_product("8x0e+8x1o", "0e+1o+2e", "0e+1o")
    poly = e.polynomial.flatten_coefficient_modes().squeeze_modes()
    f = cb.SegmentedPolynomial(poly, method="uniform_1d")
    gen = torch.Generator().manual_seed(hash((in_modes, out_mode)) % 2**31)
    batch, rows = 7, 3
    xs, idx = [], {}
    for k, mode in enumerate(in_modes):
        x, i = _make_operand(mode, poly.inputs[k].size, batch, rows, gen, dtype)
        xs.append(x)
        if i is not None:
            idx[k] = i
    has_batch = any(m != "shared" for m in in_modes)
    oshape, oidx = {}, {}
    if out_mode == "shared":
        oshape = {0: 1}
    elif out_mode == "indexed":
        if not has_batch:
            pytest.skip("an indexed output needs a batch")
        oshape = {0: rows}
        oidx = {0: torch.randint(0, rows, (batch,), generator=gen)}
    cot_rows = {"shared": 1, "batched": batch if has_batch else 1, "indexed": rows}[out_mode]
    cot = torch.randn(cot_rows, poly.outputs[0].size, generator=gen, dtype=torch.float64).to(dtype)

    ref = _derivatives(lambda *a: naive.segmented_polynomial(poly, list(a), idx, oshape, oidx)[0], xs, cot)
    dev_idx = {k: v.to(DEV) for k, v in idx.items()}
    dev_oidx = {k: v.to(DEV).to(torch.int32) for k, v in oidx.items()}
    dev_shape = {k: torch.empty(v, 1, device=DEV) for k, v in oshape.items()}
    got = _derivatives(lambda *a: f(list(a), dev_idx, dev_shape, dev_oidx)[0], [x.to(DEV) for x in xs], cot.to(DEV))
    rtol, atol = TOL[tag]
    _close(got[0], ref[0], rtol, atol, "out")
    for a, b in zip(got[1], ref[1]):
        _close(a, b, 10 * rtol, 10 * atol, "grad")
    for a, b in zip(got[2], ref[2]):
        _close(a, b, 100 * rtol, 100 * atol, "gradgrad")


def test_empty_batch():
    e = D.channelwise_tensor_product("8x0e+8x1o", "0e+1o", "0e+1o")
    f = cb.SegmentedPolynomial(e.polynomial, method="uniform_1d")
    p = e.polynomial
    xs = [torch.randn(0, o.size, device=DEV) for o in p.inputs]
    (out,) = f(xs)
    assert out.shape == (0, p.outputs[0].size)
    # empty edge list scattered into a non-empty node array gives zeros
    x1 = torch.randn(5, p.inputs[1].size, device=DEV)
    empty = torch.zeros(0, dtype=torch.int64, device=DEV)
    (out,) = f([xs[0], x1, xs[2]], {1: empty}, {0: torch.empty(5, 1, device=DEV)}, {0: empty})
    assert out.shape == (5, p.outputs[0].size) and torch.count_nonzero(out) == 0


def test_mixed_precision_inputs_float32_math():
    """bf16/fp16 inputs with float32 math: compared with the oracle run with math_dtype."""
    torch.manual_seed(3)
    e = D.channelwise_tensor_product("8x0e+8x1o", "0e+1o", "0e+1o")
    p = e.polynomial.flatten_coefficient_modes().squeeze_modes()
    for dt, tol in ((torch.bfloat16, 2e-2), (torch.float16, 3e-3)):
        xs = [torch.randn(9, o.size).to(dt) for o in p.inputs]
        f = cb.SegmentedPolynomial(p, method="uniform_1d", math_dtype=torch.float32)
        (got,) = f([x.to(DEV) for x in xs])
        assert got.dtype == dt
        (ref,) = naive.segmented_polynomial(p, [x.float() for x in xs])
        assert torch.allclose(got.float().cpu(), ref, rtol=tol, atol=tol)


def test_gather_scatter_indexing_is_exact():
    """One-hot inputs: every output entry is a single product, so the result must equal
    the oracle bit for bit, which pins the gather/scatter index arithmetic."""
    e = D.channelwise_tensor_product("4x0e", "0e", "0e")
    p = e.polynomial.flatten_coefficient_modes().squeeze_modes()
    f = cb.SegmentedPolynomial(p, method="uniform_1d")
    E, N = 257, 31
    gen = torch.Generator().manual_seed(5)
    snd, rcv = torch.randint(0, N, (E,), generator=gen), torch.arange(E) % N
    w = torch.ones(E, p.inputs[0].size)
    x1 = torch.arange(N * p.inputs[1].size, dtype=torch.float32).reshape(N, -1)
    x2 = torch.ones(E, 1)
    # make each receiver get exactly one edge contribution per slot: keep first edge per receiver
    keep = torch.zeros(E, dtype=torch.bool)
    keep[:N] = True
    x2 = x2 * keep[:, None]
    (ref,) = naive.segmented_polynomial(p, [w, x1, x2], {1: snd}, {0: N}, {0: rcv})
    (got,) = f([w.to(DEV), x1.to(DEV), x2.to(DEV)], {1: snd.to(DEV).int()}, {0: torch.empty(N, 1, device=DEV)}, {0: rcv.to(DEV).int()})
    assert torch.equal(got.cpu(), ref)


def test_fully_connected_dense_route_matches_oracle():
    """Multiplicity 16 puts the fully connected product on the dense (composite) route; it
    must agree with the CPU oracle like the flattened route does."""
    from cuequivariance_b200.fused_tp import DenseUVW

    s = "16x0e+16x1o+16x2e"
    e = D.fully_connected_tensor_product(s, s, s)
    m = cb.FullyConnectedTensorProduct(s, s, s, layout=cb.ir_mul, internal_weights=False, shared_weights=True)
    assert isinstance(m.f._program(torch.float32), DenseUVW)
    gen = torch.Generator().manual_seed(2)
    B = 24
    x1, x2 = torch.randn(B, m.irreps_in1.dim, generator=gen), torch.randn(B, m.irreps_in2.dim, generator=gen)
    w = torch.randn(1, m.weight_numel, generator=gen) / 16.0
    cot = torch.randn(B, m.irreps_out.dim, generator=gen)
    ref = _derivatives(lambda w_, a, b: naive.segmented_polynomial(e.polynomial, [w_, a, b])[0], [w, x1, x2], cot)
    got = _derivatives(lambda w_, a, b: m(a, b, w_), [w.to(DEV), x1.to(DEV), x2.to(DEV)], cot.to(DEV))
    _close(got[0], ref[0], 1e-5, 2e-6, "out")
    for a, b in zip(got[1], ref[1]):
        _close(a, b, 1e-4, 2e-5, "grad")
    for a, b in zip(got[2], ref[2]):
        _close(a, b, 1e-3, 2e-4, "gradgrad")


@pytest.mark.parametrize("fused,B", [(True, 96), (True, 300), (False, 96)])
@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float32])
def test_fully_connected_tensor_core_route(in_dtype, fused, B, monkeypatch):
    """64 channels: the tensor-core routes (bf16 operands, float32 accumulation) - ``fused``: the
    coupled operand is built on chip (four launches for forward + three gradients); otherwise
    it is written to memory and contracted by the stand-alone GEMM.  Batches that are not a
    multiple of the 128-sample tile exercise the ragged edge.  Compared with the CPU oracle
    evaluated in float32 on the same (bf16-rounded) inputs; tolerance is that of bf16 operands
    (rtol 2e-2 of the tensor's scale; the reference's own bf16 tolerance is rtol 1e-2 /
    atol 4.0, cuequivariance_torch/_tests/utils.py:282)."""
    from cuequivariance_b200 import fused_tp

    monkeypatch.setattr(fused_tp, "FUSED", fused)
    s = "64x0e+64x1o+64x2e"
    e = D.fully_connected_tensor_product(s, s, s)
    m = cb.FullyConnectedTensorProduct(s, s, s, layout=cb.ir_mul, internal_weights=False, shared_weights=True,
                                       options={"tensor_cores": True})
    gen = torch.Generator().manual_seed(22)
    x1 = torch.randn(B, m.irreps_in1.dim, generator=gen).to(in_dtype)
    x2 = torch.randn(B, m.irreps_in2.dim, generator=gen).to(in_dtype)
    w = (torch.randn(1, m.weight_numel, generator=gen) / 64.0).to(in_dtype)
    cot = torch.randn(B, m.irreps_out.dim, generator=gen)

    def grads(fn, xs, c):
        xs = [x.clone().requires_grad_(True) for x in xs]
        out = fn(*xs)
        return [out.detach()] + list(torch.autograd.grad((out.float() * c).sum(), xs))

    ref = grads(lambda w_, a, b: naive.segmented_polynomial(e.polynomial, [w_, a, b])[0], [w.float(), x1.float(), x2.float()], cot)
    profiling.reset()
    profiling.enable()
    try:
        got = grads(lambda w_, a, b: m(a, b, w_), [w.to(DEV), x1.to(DEV), x2.to(DEV)], cot.to(DEV))
        names = set(profiling.summary())
    finally:
        profiling.enable(False)
    assert profiling.launch_count >= (4 if fused else 3 * 11), "the tensor-core route did not run"
    assert ({"fctp_fused_forward", "fctp_fused_gw", "fctp_fused_gx1", "fctp_fused_gx2"} <= names) == fused, names
    for name, a, b in zip(["out", "gw", "gx1", "gx2"], got, ref):
        scale = float(b.abs().max())
        err = float((a.float().cpu() - b).abs().max())
        assert err <= 2e-2 * scale, f"{name}: max abs diff {err:.3e} at scale {scale:.3e}"


@pytest.mark.parametrize("tag", ["f64", "f32"])
@pytest.mark.parametrize("classes", [1, 3])
def test_linear_module_against_oracle(tag, classes):
    """`Linear` (surface of cuequivariance_torch/operations/linear.py:30-191) against the oracle on the
    descriptor's polynomial, with and without weight classes selected by `weight_indices`; the mul_ir
    variant must equal the ir_mul one up to the layout transposition."""
    dtype = DT[tag]
    s_in, s_out = "6x0e+5x1o+4x2e", "3x0e+7x1o+2x2e+4x3o"
    e = D.linear(s_in, s_out)
    m = cb.Linear(s_in, s_out, layout=cb.ir_mul, internal_weights=False, shared_weights=True, weight_classes=classes, dtype=dtype)
    gen = torch.Generator().manual_seed(5 + classes)
    B = 11
    x = torch.randn(B, m.irreps_in.dim, generator=gen, dtype=dtype)
    w = torch.randn(classes, m.weight_numel, generator=gen, dtype=dtype)
    cot = torch.randn(B, m.irreps_out.dim, generator=gen, dtype=dtype)
    idx = torch.randint(0, classes, (B,), generator=gen) if classes > 1 else None

    def ref_fn(w_, x_):
        return naive.segmented_polynomial(e.polynomial, [w_, x_], {0: idx} if idx is not None else {})[0]

    def got_fn(w_, x_):
        return m(x_, w_, weight_indices=idx.to(DEV) if idx is not None else None)

    ref = _derivatives(ref_fn, [w, x], cot)
    got = _derivatives(got_fn, [w.to(DEV), x.to(DEV)], cot.to(DEV))
    rtol, atol = TOL[tag]
    _close(got[0], ref[0], rtol, atol, "out")
    for a, b in zip(got[1], ref[1]):
        _close(a, b, 10 * rtol, 10 * atol, "grad")
    for a, b in zip(got[2], ref[2]):
        _close(a, b, 100 * rtol, 100 * atol, "gradgrad")
    m2 = cb.Linear(s_in, s_out, layout=cb.mul_ir, internal_weights=False, shared_weights=True, weight_classes=classes, dtype=dtype)
    to_mul_ir = cb.TransposeIrrepsLayout(s_in, source=cb.ir_mul, target=cb.mul_ir)
    back = cb.TransposeIrrepsLayout(s_out, source=cb.mul_ir, target=cb.ir_mul)
    y2 = back(m2(to_mul_ir(x.to(DEV)), w.to(DEV), weight_indices=idx.to(DEV) if idx is not None else None))
    _close(y2, got[0], rtol, atol, "mul_ir")


def test_linear_dense_route_against_oracle():
    """Multiplicities that are multiples of 32: `Linear` runs as float32-accurate tensor-core GEMMs
    (three TF32 passes).  Output and first derivatives against the oracle in float32; the same module on
    the generic kernel (dense route switched off) must agree as well."""
    from cuequivariance_b200.operations import linear as linear_mod

    s_in, s_out = "64x0e+32x1o+32x2e", "32x0e+64x1o+32x2e"
    e = D.linear(s_in, s_out)
    m = cb.Linear(s_in, s_out, layout=cb.mul_ir, internal_weights=False, shared_weights=True)
    gen = torch.Generator().manual_seed(77)
    B = 300
    x = torch.randn(B, m.irreps_in.dim, generator=gen)
    w = torch.randn(1, m.weight_numel, generator=gen)
    cot = torch.randn(B, m.irreps_out.dim, generator=gen)

    def grads(fn, xs, c):
        xs = [t.clone().requires_grad_(True) for t in xs]
        out = fn(*xs)
        return [out.detach()] + list(torch.autograd.grad((out * c).sum(), xs))

    profiling.reset()
    profiling.enable()
    try:
        got = grads(lambda w_, x_: m(x_, w_), [w.to(DEV), x.to(DEV)], cot.to(DEV))
        names = set(profiling.summary())
    finally:
        profiling.enable(False)
    assert "linear_f32x3" in names and "linear_f32x3_gx" in names, names
    old = linear_mod.DENSE_ROUTE
    linear_mod.DENSE_ROUTE = False
    try:
        gen_route = grads(lambda w_, x_: m(x_, w_), [w.to(DEV), x.to(DEV)], cot.to(DEV))
    finally:
        linear_mod.DENSE_ROUTE = old
    for name, a, b in zip(["out", "gw", "gx"], got, gen_route):
        _close(a, b, 1e-4, 2e-5, name + " (dense vs generic)")
    # oracle on the ir_mul polynomial: transpose on the device with the module's own transposes
    to_ir_mul = cb.TransposeIrrepsLayout(s_in, source=cb.mul_ir, target=cb.ir_mul)
    back = cb.TransposeIrrepsLayout(s_out, source=cb.mul_ir, target=cb.ir_mul)
    x_im = to_ir_mul(x.to(DEV)).cpu()
    ref = naive.segmented_polynomial(e.polynomial, [w, x_im])[0]
    _close(back(got[0]).cpu(), ref, 1e-5, 2e-6, "out vs oracle")


def test_equivariant_tensor_product_wrapper_matches_oracle():
    """`EquivariantTensorProduct` built from a descriptor: layout transposes of every operand around
    the executor, gather of the second input and scatter of the output, against the oracle."""
    e = D.channelwise_tensor_product("8x0e+8x1o+8x2e", "0e+1o+2e", ["0e", "1o", "2e"])
    m = cb.EquivariantTensorProduct(e, layout=cb.mul_ir)
    gen = torch.Generator().manual_seed(9)
    E, N = 40, 6
    w = torch.randn(E, e.inputs[0].dim, generator=gen)
    x1 = torch.randn(N, e.inputs[1].dim, generator=gen)
    x2 = torch.randn(E, e.inputs[2].dim, generator=gen)
    snd, rcv = torch.randint(0, N, (E,), generator=gen), torch.randint(0, N, (E,), generator=gen)
    cot = torch.randn(N, e.outputs[0].dim, generator=gen)
    blocks = [[(mu, ir.dim) for mu, ir in r.irreps] for r in e.inputs + e.outputs]

    def ref_fn(w_, a, b):
        xs = [naive.transpose_layout(t, bl, True) for t, bl in zip((w_, a, b), blocks)]
        (o,) = naive.segmented_polynomial(e.polynomial, xs, {1: snd}, {0: N}, {0: rcv})
        return naive.transpose_layout(o, blocks[3], False)

    ref = _derivatives(ref_fn, [w, x1, x2], cot)
    got = _derivatives(lambda w_, a, b: m(w_, a, b, indices={1: snd.to(DEV)}, indices_out=rcv.to(DEV), size_out=N),
                       [w.to(DEV), x1.to(DEV), x2.to(DEV)], cot.to(DEV))
    _close(got[0], ref[0], 1e-5, 2e-6, "out")
    for a, b in zip(got[1], ref[1]):
        _close(a, b, 1e-4, 2e-5, "grad")
    for a, b in zip(got[2], ref[2]):
        _close(a, b, 1e-3, 2e-4, "gradgrad")


def test_modules_survive_a_pickle_round_trip():
    """`__reduce__` rebuilds the module from (polynomial, method, math_dtype, ...), like the reference
    (cuequivariance_torch/primitives/segmented_polynomial.py:237-248): the copy must give the same bits."""
    import pickle

    e = D.channelwise_tensor_product("8x0e+8x1o", "0e+1o+2e", "0e+1o")
    f = cb.SegmentedPolynomial(e.polynomial, method="uniform_1d", math_dtype="float32", name="pickled")
    f2 = pickle.loads(pickle.dumps(f))
    assert f2.method == f.method and f2.math_dtype == f.math_dtype and f2.name == "pickled" and repr(f2) == repr(f)
    xs = [torch.randn(5, o.size, device=DEV) for o in e.polynomial.inputs]
    assert torch.equal(f(xs)[0], f2(xs)[0])
    tp = cb.ChannelWiseTensorProduct("8x0e+8x1o", "0e+1o", ["0e", "1o"], layout=cb.mul_ir, shared_weights=True, internal_weights=True, device=DEV)
    tp2 = pickle.loads(pickle.dumps(tp))
    a, b = torch.randn(5, tp.irreps_in1.dim, device=DEV), torch.randn(5, tp.irreps_in2.dim, device=DEV)
    assert torch.equal(tp(a, b), tp2(a, b))


@pytest.mark.parametrize("method", [None, "indexed_linear"])
def test_linear_weight_classes_on_grouped_gemms(method):
    """`Linear` with one weight set per class and rows sorted by class (the reference's `indexed_linear`
    situation, cuequivariance_torch/primitives/segmented_polynomial_indexed_linear.py:247-339): one float32-accurate
    tensor-core GEMM per (class, irrep pair).  Output and first derivatives against the oracle with indexed
    weights; unsorted indices take the generic kernel (default method) or raise (method="indexed_linear")."""
    s_in, s_out = "64x0e+32x1o+32x2e", "32x0e+64x1o+32x2e"
    classes, B = 5, 320
    e = D.linear(s_in, s_out)
    m = cb.Linear(s_in, s_out, layout=cb.ir_mul, internal_weights=False, shared_weights=True, weight_classes=classes, method=method)
    gen = torch.Generator().manual_seed(78)
    x = torch.randn(B, m.irreps_in.dim, generator=gen)
    w = torch.randn(classes, m.weight_numel, generator=gen)
    cot = torch.randn(B, m.irreps_out.dim, generator=gen)
    idx = torch.sort(torch.randint(0, classes - 1, (B,), generator=gen)).values     # the last class owns no row

    def grads(fn, xs, c):
        xs = [t.clone().requires_grad_(True) for t in xs]
        out = fn(*xs)
        return [out.detach()] + list(torch.autograd.grad((out * c).sum(), xs))

    ref = grads(lambda w_, x_: naive.segmented_polynomial(e.polynomial, [w_, x_], {0: idx})[0], [w, x], cot)
    profiling.reset()
    profiling.enable()
    try:
        got = grads(lambda w_, x_: m(x_, w_, weight_indices=idx.to(DEV)), [w.to(DEV), x.to(DEV)], cot.to(DEV))
        names = set(profiling.summary())
    finally:
        profiling.enable(False)
    assert {"indexed_linear_f32x3", "indexed_linear_f32x3_gx", "indexed_linear_f32x3_gw"} <= names, names
    for name, a, b in zip(["out", "grad w", "grad x"], got, ref):
        f = 1 if name == "out" else 10
        _close(a, b, f * 1e-5, f * 2e-6, name)
    shuffled = idx[torch.randperm(B, generator=gen)]
    if method == "indexed_linear":
        with pytest.raises(ValueError, match="non-sorted"):
            m(x.to(DEV), w.to(DEV), weight_indices=shuffled.to(DEV))
    else:
        (ref2,) = naive.segmented_polynomial(e.polynomial, [w, x], {0: shuffled})
        _close(m(x.to(DEV), w.to(DEV), weight_indices=shuffled.to(DEV)), ref2, 1e-5, 2e-6, "unsorted indices")


@pytest.mark.parametrize("tag", ["f64", "f32"])
@pytest.mark.parametrize("ls,normalize", [([0, 1, 2, 3], True), ([1, 3], False), ([0, 2, 4], True)])
def test_fused_spherical_harmonics_against_oracle(tag, ls, normalize):
    """The fused kernels (normalisation + all degrees in one pass; first derivative) against the oracle on the
    descriptor's polynomial; the second derivative (taken with create_graph) runs through the polynomial executor."""
    dtype = DT[tag]
    sh = cb.SphericalHarmonics(ls, normalize=normalize)
    e = D.spherical_harmonics("1o", ls)
    gen = torch.Generator().manual_seed(sum(ls))
    vec = torch.randn(257, 3, generator=gen, dtype=torch.float64).to(dtype) * 2.0
    cot = torch.randn(257, sum(2 * l + 1 for l in ls), generator=gen, dtype=torch.float64).to(dtype)

    def ref_fn(v):
        v = torch.nn.functional.normalize(v, dim=1) if normalize else v
        return naive.segmented_polynomial(e.polynomial, [v])[0]

    ref = _derivatives(ref_fn, [vec], cot)
    profiling.reset()
    profiling.enable()
    try:
        got = _derivatives(lambda v: sh(v), [vec.to(DEV)], cot.to(DEV))
        names = set(profiling.summary())
    finally:
        profiling.enable(False)
    assert {"sh_fused_forward", "sh_fused_backward"} <= names, names
    rtol, atol = TOL[tag]
    _close(got[0], ref[0], rtol, atol, "out")
    _close(got[1][0], ref[1][0], 10 * rtol, 10 * atol, "grad")
    _close(got[2][0], ref[2][0], 100 * rtol, 100 * atol, "gradgrad")


def test_index_range_debug_mode_flags_and_clamps(monkeypatch):
    """With index checking on, an out-of-range scatter index is reported through the status word (code 3) and
    clamped, so nothing faults; with valid indices the mode changes no result."""
    from cuequivariance_b200 import _lib

    monkeypatch.setattr(_lib, "CHECK_INDICES", True)
    e = D.channelwise_tensor_product("8x0e+8x1o", "0e+1o", "0e+1o")
    f = cb.SegmentedPolynomial(e.polynomial, method="uniform_1d")
    p = e.polynomial
    gen = torch.Generator().manual_seed(4)
    E, N = 50, 6
    xs = [torch.randn(E, p.inputs[0].size, generator=gen), torch.randn(N, p.inputs[1].size, generator=gen), torch.randn(E, p.inputs[2].size, generator=gen)]
    snd, rcv = torch.randint(0, N, (E,), generator=gen), torch.randint(0, N, (E,), generator=gen)
    (ref,) = naive.segmented_polynomial(p, xs, {1: snd}, {0: N}, {0: rcv})
    (got,) = f([x.to(DEV) for x in xs], {1: snd.to(DEV)}, {0: torch.empty(N, 1, device=DEV)}, {0: rcv.to(DEV)})
    _close(got, ref, 1e-5, 2e-6, "valid indices")
    _lib.check_status()
    bad = rcv.clone()
    bad[7] = N + 3
    f([x.to(DEV) for x in xs], {1: snd.to(DEV)}, {0: torch.empty(N, 1, device=DEV)}, {0: bad.to(DEV)})
    with pytest.raises(_lib.CueqError, match="status 3"):
        _lib.check_status()
    _lib.check_status()   # the word was cleared
