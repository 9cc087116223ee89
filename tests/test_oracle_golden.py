"""CPU tests: descriptors and the CPU oracle against fixtures produced by the reference."""
import numpy as np
import pytest
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import descriptors as D
from oracle import naive


def _tables_equal(g, prefix, poly, ordered=True, tol=1e-14):
    assert int(g[f"{prefix}/num_inputs"]) == poly.num_inputs
    assert int(g[f"{prefix}/num_outputs"]) == poly.num_outputs
    assert int(g[f"{prefix}/num_operations"]) == len(poly.operations)
    for b, o in enumerate(poly.operands):
        ref = g[f"{prefix}/operand{b}_segments"]
        assert ref.shape[0] == o.num_segments
        assert [tuple(r) for r in ref.tolist()] == [tuple(s) for s in o.segments]
    for k, (ope, d) in enumerate(poly.operations):
        assert tuple(g[f"{prefix}/op{k}_buffers"].tolist()) == ope.buffers
        assert str(g[f"{prefix}/op{k}_subscripts"]) == d.subscripts
        idx = g[f"{prefix}/op{k}_indices"]
        mine = d.index_table()
        if f"{prefix}/op{k}_coefficients" not in g.files:  # paths with coefficient tensors of different shapes
            assert np.array_equal(idx, mine)
            for i, p in enumerate(d.paths):
                ref = g[f"{prefix}/op{k}_coefficients_{i}"]
                assert ref.shape == p.coefficients.shape and np.abs(ref - p.coefficients).max() <= tol
            continue
        coef = g[f"{prefix}/op{k}_coefficients"]
        cmine = d.coefficient_table()
        if not ordered:
            o1 = np.lexsort(idx.T[::-1])
            o2 = np.lexsort(mine.T[::-1])
            idx, coef, mine, cmine = idx[o1], coef[o1], mine[o2], cmine[o2]
        assert np.array_equal(idx, mine)
        assert np.abs(coef - cmine).max() <= tol


def test_clebsch_gordan_tables(golden):
    g = golden("cg_so3.npz")
    for key in g.files:
        l1, l2, l3 = map(int, key.split("_"))
        mine = cb.cg.so3_clebsch_gordan(l1, l2, l3)
        assert mine.shape == g[key].shape
        assert np.abs(mine - g[key]).max() < 1e-14
        # same sparsity pattern (the flattened path lists depend on it)
        assert np.array_equal(mine != 0, g[key] != 0)


def test_clebsch_gordan_intertwines_rotations():
    # C (R1 x R2) = R3 C for rotations generated from the l=1 coupling (the identity the
    # reference tests check, cuequivariance/tests/group_theory/clebsch_gordan_test.py:23-35)
    rng = np.random.default_rng(0)
    x, y = rng.normal(size=3), rng.normal(size=3)
    c = cb.cg.so3_clebsch_gordan(1, 1, 1)[0]
    z = np.einsum("ijk,i,j->k", c, x, y)
    # l=1 (x) l=1 -> l=1 is the cross product up to scale: orthogonal to both inputs
    assert abs(z @ x) < 1e-12 and abs(z @ y) < 1e-12


DESCRIPTORS = {
    "cw_l2": lambda: D.channelwise_tensor_product("8x0e+8x1o+8x2e", "0e+1o+2e+3o", ["0e", "1o", "2e", "3o"]),
    "cw_l3": lambda: D.channelwise_tensor_product("8x0e+8x1o+8x2e+8x3o", "0e+1o+2e+3o", ["0e", "1o", "2e", "3o"]),
    "cw_mixed": lambda: D.channelwise_tensor_product("4x0e+4x1o+4x1e", "0e+1o+1e+2e", None),
    "fc": lambda: D.fully_connected_tensor_product("4x0e+4x1o+4x2e", "4x0e+4x1o+4x2e", "4x0e+4x1o+4x2e"),
    "linear": lambda: D.linear("5x0e+3x1o", "4x0e+2x1o"),
}


@pytest.mark.parametrize("name", list(DESCRIPTORS))
def test_descriptor_tables_match_reference(golden, name):
    g = golden("descriptors.npz")
    e = DESCRIPTORS[name]()
    _tables_equal(g, name, e.polynomial)
    if name.startswith("cw"):
        assert repr(e.outputs[0].irreps) == str(g[f"{name}/irreps_out"])
        flat = e.polynomial.flatten_coefficient_modes().squeeze_modes()
        _tables_equal(g, f"{name}_flat", flat)


def test_spherical_harmonics_tables_match_reference(golden):
    g = golden("descriptors.npz")
    e = D.spherical_harmonics("1o", [0, 1, 2, 3])
    _tables_equal(g, "sh", e.polynomial, ordered=False, tol=1e-13)


def _t(a, dtype=None):
    t = torch.from_numpy(np.array(a))
    return t if dtype is None else t.to(dtype)


def _derivatives(fn, inputs, cot):
    xs = [x.clone().requires_grad_(True) for x in inputs]
    out = fn(*xs)
    g1 = torch.autograd.grad((out * cot).sum(), xs, retain_graph=True, allow_unused=True)
    gg = torch.autograd.grad(out.pow(2).sum(), xs, create_graph=True, allow_unused=True)
    tot = sum(g.pow(2).sum() for g in gg if g is not None)
    g2 = torch.autograd.grad(tot, xs, allow_unused=True)
    return out.detach(), g1, g2


def _check(g, out, g1, g2, rtol, atol):
    def close(a, b, scale=1.0):
        a, b = np.asarray(a), np.asarray(b)
        assert a.shape == b.shape
        assert np.all(np.abs(a - b) <= scale * (atol + rtol * np.abs(b))), float(np.abs(a - b).max())

    close(out.numpy(), g["out"])
    for i, (a, b) in enumerate(zip(g1, g2)):
        close(a.numpy(), g[f"grad{i}"], 10)
        close(b.numpy(), g[f"gradgrad{i}"], 100)


TOL = {"f64": (1e-12, 1e-12), "f32": (1e-5, 2e-6)}


@pytest.mark.parametrize("tag", ["f64", "f32"])
@pytest.mark.parametrize("name,s1", [("cw_l2", "8x0e+8x1o+8x2e"), ("cw_l3", "8x0e+8x1o+8x2e+8x3o")])
def test_oracle_channelwise_module(golden, name, s1, tag):
    g = golden(f"{name}_module_{tag}.npz")
    e = D.channelwise_tensor_product(s1, "0e+1o+2e+3o", ["0e", "1o", "2e", "3o"])
    snd, rcv = _t(g["senders"]), _t(g["receivers"])
    N = g["x1"].shape[0]
    b1 = [(m, ir.dim) for m, ir in e.inputs[1].irreps]
    b2 = [(m, ir.dim) for m, ir in e.inputs[2].irreps]
    bo = [(m, ir.dim) for m, ir in e.outputs[0].irreps]

    def fn(w, x1, x2):
        a = naive.transpose_layout(x1, b1, True)
        b = naive.transpose_layout(x2, b2, True)
        (o,) = naive.segmented_polynomial(e.polynomial, [w, a, b], {1: snd}, {0: N}, {0: rcv})
        return naive.transpose_layout(o, bo, False)

    out, g1, g2 = _derivatives(fn, [_t(g["w"]), _t(g["x1"]), _t(g["x2"])], _t(g["cot"]))
    _check(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_oracle_uniform1d_index_modes(golden, tag):
    e = D.channelwise_tensor_product("16x0e+16x1o", "0e+1o+2e", "0e+1o")
    poly = e.polynomial.flatten_coefficient_modes().squeeze_modes()
    g = golden(f"u1d_indexed_{tag}.npz")
    ia, io = _t(g["ia"]), _t(g["io"])
    out, g1, g2 = _derivatives(
        lambda a, b, c: naive.segmented_polynomial(poly, [a, b, c], {0: ia}, {0: 3}, {0: io})[0],
        [_t(g["a"]), _t(g["b"]), _t(g["c"])], _t(g["cot"]))
    _check(g, out, g1, g2, *TOL[tag])
    g = golden(f"u1d_sum_{tag}.npz")
    a = _t(g["a"])
    out, g1, g2 = _derivatives(
        lambda b, c: naive.segmented_polynomial(poly, [a, b, c], {}, {0: 1}, {})[0], [_t(g["b"]), _t(g["c"])], _t(g["cot"]))
    _check(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_oracle_symmetric_contraction(golden, tag):
    g = golden(f"symmetric_contraction_module_{tag}.npz")
    e, _ = D.symmetric_contraction("4x0e+4x1o+4x2e+4x3o", "4x0e+4x1o", (1, 2, 3))
    sp = _t(g["species"])
    bi = [(m, ir.dim) for m, ir in e.inputs[1].irreps]
    bo = [(m, ir.dim) for m, ir in e.outputs[0].irreps]

    def fn(w, x):
        (o,) = naive.segmented_polynomial(e.polynomial, [w.flatten(1), naive.transpose_layout(x, bi, True)], {0: sp})
        return naive.transpose_layout(o, bo, False)

    out, g1, g2 = _derivatives(fn, [_t(g["weight"]), _t(g["x"])], _t(g["cot"]))
    _check(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_oracle_fully_connected(golden, tag):
    g = golden(f"fully_connected_module_{tag}.npz")
    s = "4x0e+4x1o+4x2e"
    e = D.fully_connected_tensor_product(s, s, s)
    blocks = [(m, ir.dim) for m, ir in e.inputs[1].irreps]

    def fn(w, x1, x2):
        (o,) = naive.segmented_polynomial(
            e.polynomial, [w, naive.transpose_layout(x1, blocks, True), naive.transpose_layout(x2, blocks, True)])
        return naive.transpose_layout(o, blocks, False)

    out, g1, g2 = _derivatives(fn, [_t(g["weight"]), _t(g["x1"]), _t(g["x2"])], _t(g["cot"]))
    _check(g, out, g1, g2, *TOL[tag])


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_oracle_spherical_harmonics(golden, tag):
    g = golden(f"spherical_harmonics_{tag}.npz")
    e = D.spherical_harmonics("1o", [0, 1, 2, 3])

    def fn(v):
        return naive.segmented_polynomial(e.polynomial, [torch.nn.functional.normalize(v, dim=1)])[0]

    out, g1, g2 = _derivatives(fn, [_t(g["vec"])], _t(g["cot"]))
    _check(g, out, g1, g2, *TOL[tag])
    # component normalisation: |Y_l|^2 = 2l+1 on unit vectors
    y = out.double().numpy()
    assert np.allclose((y**2).sum(1), 16.0, rtol=1e-5 if tag == "f32" else 1e-12)


@pytest.mark.parametrize("tag", ["f64", "f32"])
def test_oracle_transpose(golden, tag):
    g = golden(f"transpose_{tag}.npz")
    y = naive.transpose_layout(_t(g["x"]), [(3, 1), (5, 3), (2, 5)], True)
    assert np.array_equal(y.numpy(), g["y"])


def test_backward_polynomial_equals_autograd():
    """Derived backward polynomial, evaluated by the oracle with swapped gather/scatter
    roles, equals autograd of the forward evaluation."""
    torch.manual_seed(0)
    e = D.channelwise_tensor_product("4x0e+4x1o+4x2e", "0e+1o+2e", ["0e", "1o", "2e"])
    poly = e.polynomial.flatten_coefficient_modes().squeeze_modes()
    E, N = 30, 6
    w = torch.randn(E, poly.inputs[0].size, dtype=torch.float64, requires_grad=True)
    x1 = torch.randn(N, poly.inputs[1].size, dtype=torch.float64, requires_grad=True)
    x2 = torch.randn(E, poly.inputs[2].size, dtype=torch.float64, requires_grad=True)
    snd, rcv = torch.randint(0, N, (E,)), torch.randint(0, N, (E,))
    (out,) = naive.segmented_polynomial(poly, [w, x1, x2], {1: snd}, {0: N}, {0: rcv})
    cot = torch.randn_like(out)
    ref = torch.autograd.grad((out * cot).sum(), [w, x1, x2])
    bwd = poly.backward([True, True, True], [True])
    got = naive.segmented_polynomial(
        bwd, [w.detach(), x1.detach(), x2.detach(), cot], {1: snd, 3: rcv}, {1: N}, {1: snd})
    for a, b in zip(got, ref):
        assert torch.allclose(a, b, rtol=1e-12, atol=1e-12)
