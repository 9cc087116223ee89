"""GPU parity of the specialised channelwise kernels against the CPU oracle: layouts,
sorted and unsorted receivers, with and without gather/scatter, channel counts that use one
lane, a full warp and two channel blocks, and every gradient mask.

float32 tolerance: |a-b| <= rtol*|b| + atol*scale with rtol 1e-5, atol 2e-6 on outputs (x10
on gradients) and scale = max(1, max|b|): entries are sums of hundreds to thousands of
products that partly cancel, so the absolute term has to be in units of the tensor's
magnitude (the float32 oracle itself differs from the float64 one by that much)."""
import numpy as np
import pytest
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import descriptors as D, profiling
from oracle import naive

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
FILTER = ["0e", "1o", "2e", "3o"]


def _sh(vec):
    e = D.spherical_harmonics("1o", [0, 1, 2, 3])
    return naive.segmented_polynomial(e.polynomial, [torch.nn.functional.normalize(vec, dim=1)])[0]


def _close(a, b, rtol, atol, what):
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    excess = (a - b).abs() - (atol * max(1.0, float(b.abs().max())) + rtol * b.abs())
    assert excess.max() <= 0, f"{what}: max abs diff {(a - b).abs().max():.3e}"


def _oracle(e, layout, snd, rcv, N):
    b1 = [(m, ir.dim) for m, ir in e.inputs[1].irreps]
    bo = [(m, ir.dim) for m, ir in e.outputs[0].irreps]

    def fn(w, x1, x2):
        a = naive.transpose_layout(x1, b1, True) if layout is cb.mul_ir else x1
        ii = {1: snd} if snd is not None else {}
        oi = {0: rcv} if rcv is not None else {}
        os_ = {0: N} if rcv is not None else {}
        (o,) = naive.segmented_polynomial(e.polynomial, [w, a, x2], ii, os_, oi)
        return naive.transpose_layout(o, bo, False) if layout is cb.mul_ir else o

    return fn


def _grads(fn, xs, cot, mask=(True, True, True)):
    xs = [x.clone().requires_grad_(m) for x, m in zip(xs, mask)]
    out = fn(*xs)
    gs = torch.autograd.grad((out * cot).sum(), [x for x, m in zip(xs, mask) if m])
    return out.detach(), list(gs)


@pytest.mark.parametrize("layout", [cb.mul_ir, cb.ir_mul])
@pytest.mark.parametrize("mul,irreps1", [(4, "l2"), (32, "l3"), (128, "l3"), (256, "l2")])
@pytest.mark.parametrize("sorted_receivers", [True, False])
@pytest.mark.parametrize("cpl,staging,variant", [(2, 0, 1), (4, 0, 1), (2, 1, 1), (4, 1, 1), (0, 0, 2), (0, 0, 3), (0, 0, 0)])  # variant: backward kernel (1 = warp per receiver, 2 = thread block per receiver, 3 = 2 with bulk reductions)
def test_channelwise_kernels_match_oracle(layout, mul, irreps1, sorted_receivers, cpl, staging, variant, monkeypatch):
    from cuequivariance_b200 import channelwise

    if variant == 3 and mul % 128:
        pytest.skip("the bulk-reduction backward needs a multiple of 128 channels")

    monkeypatch.setattr(channelwise, "CHANNELS_PER_LANE", cpl)
    monkeypatch.setattr(channelwise, "STAGING", staging)
    monkeypatch.setattr(channelwise, "BWD_VARIANT", variant)
    s1 = "+".join(f"{mul}x{ir}" for ir in (["0e", "1o", "2e"] if irreps1 == "l2" else ["0e", "1o", "2e", "3o"]))
    e = D.channelwise_tensor_product(s1, "0e+1o+2e+3o", FILTER)
    m = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", FILTER, layout=layout, shared_weights=False, internal_weights=False)
    gen = torch.Generator().manual_seed(mul * 7 + sorted_receivers)
    E, N = (300, 37) if mul <= 32 else (90, 11)
    x1 = torch.randn(N, m.irreps_in1.dim, generator=gen)
    x2 = _sh(torch.randn(E, 3, generator=gen))
    w = torch.randn(E, m.weight_numel, generator=gen)
    snd = torch.randint(0, N, (E,), generator=gen)
    rcv = torch.randint(0, N - 2, (E,), generator=gen)  # the last receivers get no edge
    if sorted_receivers:
        rcv = torch.sort(rcv).values
    cot = torch.randn(N, m.irreps_out.dim, generator=gen)
    ref_out, ref_g = _grads(_oracle(e, layout, snd, rcv, N), [w, x1, x2], cot)
    profiling.reset()
    d = lambda t: t.to(DEV)  # noqa: E731
    out, g = _grads(lambda w_, a, b: m(a, b, w_, indices_1=d(snd).int(), indices_out=d(rcv), size_out=N),
                    [d(w), d(x1), d(x2)], d(cot))
    n_launch = len(m.f._program(torch.float32)._special.plan.groups)
    assert n_launch >= (3 if irreps1 == "l2" else 4)
    assert profiling.launch_count == 2 * n_launch, "the specialised kernels did not run"
    _close(out, ref_out, 1e-5, 2e-6, "out")
    for name, a, b in zip(["gw", "gx1", "gx2"], g, ref_g):
        _close(a, b, 1e-4, 2e-5, name)


@pytest.mark.parametrize("mul", [16, 128])   # 128 channels: the block-per-receiver backward and its variants without x2 gradient
@pytest.mark.parametrize("mask", [(True, False, False), (False, True, False), (False, False, True), (True, False, True), (True, True, False)])
def test_channelwise_gradient_masks(mask, mul):
    s1 = f"{mul}x0e+{mul}x1o+{mul}x2e+{mul}x3o"
    e = D.channelwise_tensor_product(s1, "0e+1o+2e+3o", FILTER)
    m = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    gen = torch.Generator().manual_seed(11)
    E, N = 120, 13
    x1, x2 = torch.randn(N, m.irreps_in1.dim, generator=gen), _sh(torch.randn(E, 3, generator=gen))
    w = torch.randn(E, m.weight_numel, generator=gen)
    snd, rcv = torch.randint(0, N, (E,), generator=gen), torch.randint(0, N, (E,), generator=gen)
    cot = torch.randn(N, m.irreps_out.dim, generator=gen)
    ref_out, ref_g = _grads(_oracle(e, cb.mul_ir, snd, rcv, N), [w, x1, x2], cot, mask)
    d = lambda t: t.to(DEV)  # noqa: E731
    out, g = _grads(lambda w_, a, b: m(a, b, w_, indices_1=d(snd), indices_out=d(rcv), size_out=N), [d(w), d(x1), d(x2)], d(cot), mask)
    _close(out, ref_out, 1e-5, 2e-6, "out")
    for a, b in zip(g, ref_g):
        _close(a, b, 1e-4, 2e-5, "grad")


def test_channelwise_without_indices():
    """No gather, no scatter: every edge is its own receiver (batched x1 and output)."""
    s1 = "8x0e+8x1o+8x2e+8x3o"
    e = D.channelwise_tensor_product(s1, "0e+1o+2e+3o", FILTER)
    m = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", FILTER, layout=cb.ir_mul, shared_weights=False, internal_weights=False)
    gen = torch.Generator().manual_seed(21)
    E = 70
    x1, x2 = torch.randn(E, m.irreps_in1.dim, generator=gen), _sh(torch.randn(E, 3, generator=gen))
    w = torch.randn(E, m.weight_numel, generator=gen)
    cot = torch.randn(E, m.irreps_out.dim, generator=gen)
    ref_out, ref_g = _grads(_oracle(e, cb.ir_mul, None, None, E), [w, x1, x2], cot)
    d = lambda t: t.to(DEV)  # noqa: E731
    profiling.reset()
    out, g = _grads(lambda w_, a, b: m(a, b, w_), [d(w), d(x1), d(x2)], d(cot))
    assert profiling.launch_count == 2 * len(m.f._program(torch.float32)._special.plan.groups)
    _close(out, ref_out, 1e-5, 2e-6, "out")
    for a, b in zip(g, ref_g):
        _close(a, b, 1e-4, 2e-5, "grad")


def test_linearity_at_scale():
    """Size-independent property at a larger size: out(w1 + w2) = out(w1) + out(w2) and the
    scatter conserves the total (sum over receivers = sum over edges of per-edge outputs)."""
    s1 = "128x0e+128x1o+128x2e+128x3o"
    m = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    gen = torch.Generator(device=DEV).manual_seed(5)
    E, N = 20000, 700
    x1 = torch.randn(N, m.irreps_in1.dim, generator=gen, device=DEV)
    x2 = torch.randn(E, 16, generator=gen, device=DEV)
    w1 = torch.randn(E, m.weight_numel, generator=gen, device=DEV)
    w2 = torch.randn(E, m.weight_numel, generator=gen, device=DEV)
    snd = torch.randint(0, N, (E,), generator=gen, device=DEV)
    rcv = torch.sort(torch.randint(0, N, (E,), generator=gen, device=DEV)).values
    f = lambda w: m(x1, x2, w, indices_1=snd, indices_out=rcv, size_out=N)  # noqa: E731
    a, b, c = f(w1), f(w2), f(w1 + w2)
    assert torch.allclose(a + b, c, rtol=1e-4, atol=2e-4)
    per_edge = m(x1, x2, w1, indices_1=snd)           # no scatter
    assert torch.allclose(per_edge.double().sum(0), a.double().sum(0), rtol=1e-6, atol=1e-3)
    # run-to-run reproducibility of the forward (no atomics on that path)
    assert torch.equal(f(w1), a)


def test_force_training_chain_float32_kernels_vs_float64_executor():
    """Config-4 pattern at 65,536 edges: energy = sum of the 0e outputs, forces-like first
    derivatives, then the gradient of their squared norm (double backward).  The float32
    specialised kernels (first order + composed second order) are checked against the same
    chain evaluated in float64 by the generic executor: an independent code path, itself
    pinned on the reference fixtures and the CPU oracle at small sizes."""
    s1 = "+".join(f"32x{ir}" for ir in FILTER)
    E, N = 65536, 4096
    tp = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", FILTER, layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    gen = torch.Generator(device=DEV).manual_seed(44)
    x1 = torch.randn(N, tp.irreps_in1.dim, generator=gen, device=DEV, dtype=torch.float64)
    x2 = torch.randn(E, 16, generator=gen, device=DEV, dtype=torch.float64)
    w = torch.randn(E, tp.weight_numel, generator=gen, device=DEV, dtype=torch.float64)
    snd = torch.randint(0, N, (E,), generator=gen, device=DEV, dtype=torch.int32)
    rcv = torch.sort(torch.randint(0, N, (E,), generator=gen, device=DEV, dtype=torch.int32)).values

    def chain(dtype):
        a, b, c = (t.to(dtype).clone().requires_grad_(True) for t in (x1, x2, w))
        out = tp(a, b, c, indices_1=snd, indices_out=rcv, size_out=N)
        energy = out[:, : 4 * 32].sum()
        ga, gb, gc = torch.autograd.grad(energy, (a, b, c), create_graph=True)
        loss = gb.pow(2).sum() + 1e-3 * ga.pow(2).sum() + 1e-3 * gc.pow(2).sum()
        return [out.detach(), ga.detach(), gb.detach(), gc.detach()] + [t.detach() for t in torch.autograd.grad(loss, (a, b, c))]

    profiling.reset()
    got = chain(torch.float32)
    assert profiling.launch_count > 0
    ref = chain(torch.float64)
    for name, a, b in zip(["out", "gx1", "gx2", "gw", "ggx1", "ggx2", "ggw"], got, ref):
        scale = max(1.0, float(b.abs().max()))
        err = float((a.double() - b).abs().max())
        assert err <= 2e-5 * scale, f"{name}: max abs diff {err:.3e} at scale {scale:.3e}"
