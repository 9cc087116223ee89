"""CPU checks of the test infrastructure itself: the numpy evaluator (an implementation that
shares no code with the torch oracle) must agree with `oracle/naive.py`, and the chunked
runner must agree with the one-shot evaluation, values and gradients."""
import itertools

import numpy as np
import pytest
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import descriptors as D
from oracle import chunked, evaluate_numpy, naive


def _rand(shape, gen):
    return torch.randn(*shape, generator=gen, dtype=torch.float64)


@pytest.mark.parametrize("name", ["channelwise", "channelwise_flat", "fully_connected", "symmetric_contraction", "linear", "spherical_harmonics"])
def test_numpy_evaluator_agrees_with_the_torch_oracle(name):
    gen = torch.Generator().manual_seed(7)
    if name.startswith("channelwise"):
        p = D.channelwise_tensor_product("3x0e+3x1o+3x2e", "0e+1o+2e", ["0e", "1o", "2e"]).polynomial
        if name.endswith("flat"):
            p = p.flatten_coefficient_modes().squeeze_modes()
    elif name == "fully_connected":
        p = D.fully_connected_tensor_product("2x0e+3x1o", "2x0e+2x1o", "3x0e+2x1o").polynomial
    elif name == "symmetric_contraction":
        p = D.symmetric_contraction("2x0e+2x1o", "2x0e+2x1o", (1, 2, 3))[0].polynomial
    elif name == "linear":
        p = D.linear("3x0e+2x1o", "4x0e+5x1o").polynomial
    else:
        p = D.spherical_harmonics("1o", [0, 1, 2, 3]).polynomial
    B, R = 9, 4
    for modes in itertools.product(["batched", "indexed", "shared"], repeat=min(2, len(p.inputs))):
        modes = list(modes) + ["batched"] * (len(p.inputs) - len(modes))
        xs, idx = [], {}
        for k, (op, mode) in enumerate(zip(p.inputs, modes)):
            rows = {"batched": B, "indexed": R, "shared": 1}[mode]
            xs.append(_rand((rows, op.size), gen))
            if mode == "indexed":
                idx[k] = torch.randint(0, R, (B,), generator=gen)
        for out_mode in ("plain", "scatter", "sum"):
            has_batch = any(m != "shared" for m in modes)
            if out_mode == "scatter" and not has_batch:
                continue
            orow = {} if out_mode == "plain" else ({0: R} if out_mode == "scatter" else {0: 1})
            oidx = {0: torch.randint(0, R, (B,), generator=gen)} if out_mode == "scatter" else {}
            a = naive.segmented_polynomial(p, xs, idx, orow, oidx)
            b = evaluate_numpy.evaluate(p, [x.numpy() for x in xs], {k: v.numpy() for k, v in idx.items()}, orow,
                                        {k: v.numpy() for k, v in oidx.items()})
            for u, v in zip(a, b):
                assert u.shape == v.shape
                assert np.abs(u.numpy() - v).max() <= 1e-12 * max(1.0, np.abs(v).max()), (name, modes, out_mode)


def test_chunked_runner_equals_one_shot_evaluation():
    e = D.channelwise_tensor_product("4x0e+4x1o+4x2e", "0e+1o+2e", ["0e", "1o", "2e"])
    p = e.polynomial
    gen = torch.Generator().manual_seed(0)
    E, N = 50, 7
    w, x1, x2 = _rand((E, p.inputs[0].size), gen), _rand((N, p.inputs[1].size), gen), _rand((E, p.inputs[2].size), gen)
    snd, rcv = torch.randint(0, N, (E,), generator=gen), torch.randint(0, N, (E,), generator=gen)
    cot = _rand((N, p.outputs[0].size), gen)
    (a,) = naive.segmented_polynomial(p, [w, x1, x2], {1: snd}, {0: N}, {0: rcv})
    (b,) = chunked.forward(p, [w, x1, x2], {1: snd}, {0: N}, {0: rcv}, E, chunk=16)
    assert (a - b).abs().max() < 1e-13

    def fn(rows, whole):
        w_, x2_, s_, r_ = rows
        (o,) = naive.segmented_polynomial(p, [w_, whole[0], x2_], {1: s_}, {0: N}, {0: r_})
        return (o * cot).sum()

    tot, g_rows, g_whole = chunked.value_and_grads(fn, [w, x2, snd, rcv], [x1], E, chunk=16)
    xs = [t.clone().requires_grad_(True) for t in (w, x1, x2)]
    (o,) = naive.segmented_polynomial(p, xs, {1: snd}, {0: N}, {0: rcv})
    gs = torch.autograd.grad((o * cot).sum(), xs)
    assert abs(float(tot) - float((o * cot).sum())) < 1e-10
    assert (g_rows[0] - gs[0]).abs().max() < 1e-13 and (g_rows[1] - gs[2]).abs().max() < 1e-13
    assert (g_whole[0] - gs[1]).abs().max() < 1e-12 and g_rows[2] is None and g_rows[3] is None
