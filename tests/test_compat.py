"""The stand-in for the closed `cuequivariance_ops_torch` package: the registered op
`torch.ops.cuequivariance.uniform_1d` called with the argument lists the reference front-end
builds (cuequivariance_torch/primitives/segmented_polynomial_uniform_1d.py:242-316)."""
import os
import sys

import pytest
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import compat
from cuequivariance_b200.executor import Uniform1dProgram
from oracle import naive

# the reference checkout, when present, sits next to this repository
REFERENCE = os.environ.get("CUEQ_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))


def _call_like_the_frontend(prog, inputs, input_indices, output_shapes, output_indices, math_dtype):
    """Re-states the packing of SegmentedPolynomialFromUniform1dJit.forward."""
    compat.install()
    from cuequivariance_ops_torch.uniform_1d import BATCH_DIM_AUTO, BATCH_DIM_BATCHED, BATCH_DIM_INDEXED, BATCH_DIM_SHARED

    s = prog.serialised()
    n_in, n_out = s["num_inputs"], s["num_outputs"]
    batch_dim = [BATCH_DIM_AUTO] * (n_in + n_out)
    index_buffer = [-1] * (n_in + n_out)
    tensors, num_index = list(inputs), 0
    for k, idx in input_indices.items():
        batch_dim[k] = BATCH_DIM_INDEXED
        tensors.append(idx)
        index_buffer[k] = num_index
        num_index += 1
        index_buffer.append(inputs[k].shape[0])
    for k, idx in output_indices.items():
        batch_dim[k + n_in] = BATCH_DIM_INDEXED
        tensors.append(idx)
        index_buffer[k + n_in] = num_index
        num_index += 1
        index_buffer.append(output_shapes[k])
    batch_size = BATCH_DIM_AUTO
    for k, rows in output_shapes.items():
        if batch_dim[k + n_in] == BATCH_DIM_AUTO:
            if rows == 1:
                batch_dim[k + n_in] = BATCH_DIM_SHARED
            else:
                batch_dim[k + n_in] = BATCH_DIM_BATCHED
                batch_size = rows
    starts_i = [0]
    starts_c = [0]
    for n_opnd, n_path in zip(s["num_operands"], s["num_paths"]):
        starts_i.append(starts_i[-1] + n_opnd * n_path)
        starts_c.append(starts_c[-1] + n_path)
    return torch.ops.cuequivariance.uniform_1d(
        "test", math_dtype, s["operand_extent"], n_in, n_out, num_index, s["buffer_dim"], s["buffer_num_segments"],
        batch_dim, index_buffer, list(range(n_in)) + [0] * n_out, s["num_operations"], s["num_operands"], s["operations"],
        s["num_paths"], starts_i[:-1], starts_c[:-1], s["path_indices"], s["path_coefficients"], batch_size, tensors)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_registered_op_matches_oracle_with_gradients(dtype):
    dev = "cuda:0"
    e = cb.descriptors.channelwise_tensor_product("16x0e+16x1o", "0e+1o+2e", "0e+1o")
    poly = e.polynomial.flatten_coefficient_modes().squeeze_modes()
    prog = Uniform1dProgram(poly, dtype)
    gen = torch.Generator().manual_seed(1)
    Z, R, N = 11, 4, 5
    a = torch.randn(R, poly.inputs[0].size, generator=gen, dtype=torch.float64).to(dtype)
    b = torch.randn(Z, poly.inputs[1].size, generator=gen, dtype=torch.float64).to(dtype)
    c = torch.randn(1, poly.inputs[2].size, generator=gen, dtype=torch.float64).to(dtype)
    ia, io = torch.randint(0, R, (Z,), generator=gen), torch.randint(0, N, (Z,), generator=gen)
    cot = torch.randn(N, poly.outputs[0].size, generator=gen, dtype=torch.float64).to(dtype)

    def run(fn, xs, cot):
        xs = [x.clone().requires_grad_(True) for x in xs]
        (out,) = fn(xs)
        return [out.detach()] + list(torch.autograd.grad((out * cot).sum(), xs))

    ref = run(lambda xs: naive.segmented_polynomial(poly, xs, {0: ia}, {0: N}, {0: io}), [a, b, c], cot)
    got = run(lambda xs: _call_like_the_frontend(prog, xs, {0: ia.to(dev)}, {0: N}, {0: io.to(dev)}, dtype),
              [a.to(dev), b.to(dev), c.to(dev)], cot.to(dev))
    tol = dict(rtol=1e-12, atol=1e-12) if dtype == torch.float64 else dict(rtol=1e-4, atol=1e-4)
    for x, y in zip(got, ref):
        assert torch.allclose(x.cpu(), y, **tol)


@pytest.mark.gpu
def test_segmented_transpose_stand_in(golden):
    compat.install()
    from cuequivariance_ops_torch import segmented_transpose

    g = golden("transpose_f32.npz")
    x = torch.from_numpy(g["x"]).cuda()
    info = torch.tensor([[3, 5, 3, -1], [18, 2, 5, -1]], dtype=torch.int32, device="cuda")  # 1x blocks are left out
    y = segmented_transpose(x, info, True)
    assert torch.equal(y.cpu(), torch.from_numpy(g["y"]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("subscripts", [("uv", "u", "v"), ("uv", "v", "u"), ("u", "uv", "v"), ("u", "vu", "v"),
                                        ("u", "v", "uv"), ("u", "v", "vu")])
def test_indexed_linear_stand_in(subscripts, dtype):
    """The six argument patterns the reference front-end uses
    (cuequivariance_torch/primitives/segmented_polynomial_indexed_linear.py:345-398) against float64 einsum over
    rows expanded by class, with first derivatives and one second derivative."""
    compat.install()
    from cuequivariance_ops_torch import indexed_linear

    dev = "cuda:0"
    gen = torch.Generator().manual_seed(7)
    u, v, C = 12, 20, 4
    counts = torch.tensor([5, 0, 9, 3], dtype=torch.int32)
    Z = int(counts.sum())
    cls = torch.repeat_interleave(torch.arange(C), counts.long())
    dim = {"u": u, "v": v}
    sa, sb, so = subscripts

    def make(sub):
        return torch.randn(*([C] if len(sub) == 2 else [Z]), *[dim[ch] for ch in sub], generator=gen, dtype=torch.float64)

    a, b = make(sa), make(sb)
    cot = make(so)

    def expand(t, sub):
        return t[cls] if len(sub) == 2 else t

    def ref(a_, b_):
        if len(so) == 2:
            rows = torch.einsum(f"z{sa},z{sb}->z{so}", a_, b_)
            return 0.7 * torch.zeros(C, dim[so[0]], dim[so[1]], dtype=a_.dtype).index_add_(0, cls, rows)
        return 0.7 * torch.einsum(f"z{sa},z{sb}->z{so}", expand(a_, sa), expand(b_, sb))

    def got(a_, b_):
        return indexed_linear(a_, b_, counts.to(dev), u, v, C, Z, subscripts, torch.tensor(0.7, dtype=torch.float64))

    def derivatives(fn, xs, c):
        xs = [x.clone().requires_grad_(True) for x in xs]
        out = fn(*xs)
        g = torch.autograd.grad((out * c).sum(), xs, create_graph=True)
        gg = torch.autograd.grad((g[0] ** 2).sum(), xs[1])      # through the gradient of the first argument
        return [out.detach(), g[0].detach(), g[1].detach(), gg[0]]

    want = derivatives(ref, [a, b], cot)
    have = derivatives(got, [a.to(dev).to(dtype), b.to(dev).to(dtype)], cot.to(dev).to(dtype))
    tol = 1e-11 if dtype == torch.float64 else 2e-4
    for w_, h_ in zip(want, have):
        assert h_.shape == w_.shape
        assert (h_.cpu().double() - w_).abs().max() <= tol * max(1.0, float(w_.abs().max()))


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="reference checkout not present")
def test_unmodified_reference_frontend_dispatches_to_the_stand_in():
    """Runs in a subprocess so that the reference import does not leak into other tests."""
    import subprocess

    code = f"""
import sys, types, torch
m = types.ModuleType('opt_einsum'); m.contract_path = lambda s, *a, **k: ([(0, 1)] * (len(a) - 1), types.SimpleNamespace(naive_cost=1, opt_cost=1))
sys.modules['opt_einsum'] = m
sys.path[:0] = ['{REFERENCE}/cuequivariance', '{REFERENCE}/cuequivariance_torch', '{os.path.dirname(os.path.dirname(os.path.abspath(__file__)))}']
from cuequivariance_b200 import compat
compat.install()
import cuequivariance as cue, cuequivariance_torch as cuet
e = cue.descriptors.channelwise_tensor_product(cue.Irreps('O3', '16x0e+16x1o'), cue.Irreps('O3', '0e+1o+2e'), cue.Irreps('O3', '0e+1o'))
f = cuet.SegmentedPolynomial(e.polynomial, method='uniform_1d')
assert type(f.m).__name__ == 'SegmentedPolynomialFromUniform1dJit', type(f.m)
try:
    f([torch.randn(3, o.size) for o in e.polynomial.inputs])
except RuntimeError as ex:
    assert 'no CPU fallback' in str(ex), ex
    print('DISPATCHED')
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert "DISPATCHED" in r.stdout, r.stdout + r.stderr
