"""Regenerates the golden fixtures in this directory by running the REFERENCE.

Run in a container that has the reference checkout (it is not needed at test time):

    python tests/golden/make_golden.py /path/to/reference

Every fixture is produced by the reference's own code on its naive torch path
(``method="naive"``), on CPU, from seeded inputs; the ``.npz`` files hold the inputs, the
outputs, first and second derivatives, and (for descriptor checks) the reference's
segment/path tables.  The tests compare this repository's descriptors, CPU oracle and
CUDA kernels with them.
"""
import sys
import types

import numpy as np
import torch


def _import_reference(root):
    # the reference imports opt_einsum for flop counting only; a stub (installed AFTER torch
    # is imported, so torch.einsum keeps its default contraction order) is enough.
    if "opt_einsum" not in sys.modules:
        m = types.ModuleType("opt_einsum")

        def contract_path(subscripts, *shapes, **kw):
            info = types.SimpleNamespace(naive_cost=1, opt_cost=1)
            return [(0, 1)] * (len(shapes) - 1), info

        m.contract_path = contract_path
        sys.modules["opt_einsum"] = m
    sys.path.insert(0, f"{root}/cuequivariance")
    sys.path.insert(0, f"{root}/cuequivariance_torch")
    import cuequivariance as cue
    import cuequivariance_torch as cuet

    return cue, cuet


def randn(seed, *shape, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64).to(dtype)


def randint(seed, hi, n):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, hi, (n,), generator=g, dtype=torch.int64)


def tables(poly):
    """Segment/path tables of a cue.SegmentedPolynomial as plain arrays."""
    out = {"num_inputs": np.int64(poly.num_inputs), "num_outputs": np.int64(poly.num_outputs),
           "num_operations": np.int64(len(poly.operations))}
    for b, o in enumerate(poly.operands):
        out[f"operand{b}_segments"] = np.array([list(s) for s in o.segments], dtype=np.int64).reshape(o.num_segments, o.ndim)
    for k, (ope, d) in enumerate(poly.operations):
        out[f"op{k}_buffers"] = np.array(ope.buffers, dtype=np.int64)
        out[f"op{k}_subscripts"] = np.array(str(d.subscripts))
        out[f"op{k}_indices"] = np.array([p.indices for p in d.paths], dtype=np.int64).reshape(d.num_paths, d.num_operands)
        if d.num_paths and all(p.coefficients.shape == d.paths[0].coefficients.shape for p in d.paths):
            out[f"op{k}_coefficients"] = np.stack([p.coefficients for p in d.paths])
        else:
            for i, p in enumerate(d.paths):
                out[f"op{k}_coefficients_{i}"] = p.coefficients
    return out


def derivatives(fn, inputs, cot_seed):
    """out, vjp w.r.t. every input for a random cotangent, and the reference tests' second
    order check: grads of sum(out^2) with create_graph, then sum(grad^2) backpropagated."""
    xs = [x.clone().requires_grad_(True) for x in inputs]
    out = fn(*xs)
    cot = randn(cot_seed, *out.shape, dtype=out.dtype)
    g1 = torch.autograd.grad((out * cot).sum(), xs, retain_graph=True, allow_unused=True)
    gg = torch.autograd.grad(out.pow(2).sum(), xs, create_graph=True, allow_unused=True)
    tot = sum(g.pow(2).sum() for g in gg if g is not None)
    g2 = torch.autograd.grad(tot, xs, allow_unused=True)
    res = {"out": out.detach().numpy(), "cot": cot.numpy()}
    for i, (a, b) in enumerate(zip(g1, g2)):
        res[f"grad{i}"] = a.detach().numpy() if a is not None else np.zeros(0)
        res[f"gradgrad{i}"] = b.detach().numpy() if b is not None else np.zeros(0)
    return res


def main(root, outdir):
    cue, cuet = _import_reference(root)
    torch.set_num_threads(8)

    # ---- Clebsch-Gordan tables -------------------------------------------------------
    cg = {}
    for l1 in range(5):
        for l2 in range(5):
            for l3 in range(abs(l1 - l2), min(l1 + l2, 4) + 1):
                cg[f"{l1}_{l2}_{l3}"] = cue.SO3.clebsch_gordan(cue.SO3(l1), cue.SO3(l2), cue.SO3(l3))
    np.savez_compressed(f"{outdir}/cg_so3.npz", **cg)

    # ---- descriptor tables -----------------------------------------------------------
    desc = {}
    O3 = lambda s: cue.Irreps("O3", s)  # noqa: E731
    for name, e in {
        "cw_l2": cue.descriptors.channelwise_tensor_product(O3("8x0e+8x1o+8x2e"), O3("0e+1o+2e+3o"), ["0e", "1o", "2e", "3o"]),
        "cw_l3": cue.descriptors.channelwise_tensor_product(O3("8x0e+8x1o+8x2e+8x3o"), O3("0e+1o+2e+3o"), ["0e", "1o", "2e", "3o"]),
        "cw_mixed": cue.descriptors.channelwise_tensor_product(O3("4x0e+4x1o+4x1e"), O3("0e+1o+1e+2e"), None),
        "fc": cue.descriptors.fully_connected_tensor_product(O3("4x0e+4x1o+4x2e"), O3("4x0e+4x1o+4x2e"), O3("4x0e+4x1o+4x2e")),
        "linear": cue.descriptors.linear(O3("5x0e+3x1o"), O3("4x0e+2x1o")),
        "sh": cue.descriptors.spherical_harmonics(cue.O3(1, -1), [0, 1, 2, 3]),
    }.items():
        for k, v in tables(e.polynomial).items():
            desc[f"{name}/{k}"] = v
        if name.startswith("cw"):
            flat = e.polynomial.flatten_coefficient_modes().squeeze_modes()
            for k, v in tables(flat).items():
                desc[f"{name}_flat/{k}"] = v
            bwd, _ = flat.backward([True, True, True], [True])
            for k, v in tables(bwd).items():
                desc[f"{name}_flat_bwd/{k}"] = v
            desc[f"{name}/irreps_out"] = np.array(str(e.outputs[0].irreps))
    np.savez_compressed(f"{outdir}/descriptors.npz", **desc)

    # ---- symmetric contraction table (mul independent) ----------------------------------
    from cuequivariance.group_theory.experimental.mace import symmetric_contraction as mace_sc

    e, proj = mace_sc(O3("2x0e+2x1o+2x2e+2x3o"), O3("2x0e+2x1o"), [1, 2, 3])
    sc = tables(e.polynomial)
    sc["projection"] = proj
    np.savez_compressed(f"{outdir}/symmetric_contraction_l3_to_l1_deg3.npz", **sc)

    for dtype, tag in [(torch.float64, "f64"), (torch.float32, "f32")]:
        # ---- channelwise module, mul_ir layout, gather + scatter -------------------------
        for name, s1, mul_note in [("cw_l2", "8x0e+8x1o+8x2e", 8), ("cw_l3", "8x0e+8x1o+8x2e+8x3o", 8)]:
            E, N = 96, 11
            m = cuet.ChannelWiseTensorProduct(O3(s1), O3("0e+1o+2e+3o"), ["0e", "1o", "2e", "3o"], layout=cue.mul_ir,
                                              shared_weights=False, internal_weights=False, method="naive")
            x1 = randn(100, N, m.irreps_in1.dim, dtype=dtype)
            vec = randn(101, E, 3)
            x2 = cuet.SphericalHarmonics([0, 1, 2, 3], normalize=True, method="naive")(vec.to(dtype))
            w = randn(102, E, m.weight_numel, dtype=dtype)
            snd, rcv = randint(103, N, E), randint(104, N, E)
            res = derivatives(lambda w_, a, b: m(a, b, w_, indices_1=snd, indices_out=rcv, size_out=N), [w, x1, x2], 105)
            np.savez_compressed(f"{outdir}/{name}_module_{tag}.npz", w=w.numpy(), x1=x1.numpy(), x2=x2.detach().numpy(),
                                vec=vec.numpy(), senders=snd.numpy(), receivers=rcv.numpy(), **res)

        # ---- the reference executor tests' polynomial, raw executor call, all index modes -------
        e = cue.descriptors.channelwise_tensor_product(O3("16x0e+16x1o"), O3("0e+1o+2e"), O3("0e+1o"))
        poly = e.polynomial.flatten_coefficient_modes().squeeze_modes()
        f = cuet.SegmentedPolynomial(poly, method="naive")
        Z, R = 10, 4
        a = randn(110, R, poly.inputs[0].size, dtype=dtype)     # indexed weights
        b = randn(111, Z, poly.inputs[1].size, dtype=dtype)     # batched
        c = randn(112, 1, poly.inputs[2].size, dtype=dtype)     # shared
        ia, io = randint(113, R, Z), randint(114, 3, Z)
        res = derivatives(lambda a_, b_, c_: f([a_, b_, c_], {0: ia}, {0: torch.empty(3, 1)}, {0: io})[0], [a, b, c], 115)
        np.savez_compressed(f"{outdir}/u1d_indexed_{tag}.npz", a=a.numpy(), b=b.numpy(), c=c.numpy(), ia=ia.numpy(), io=io.numpy(), **res)
        res = derivatives(lambda b_, c_: f([a[:1], b_, c_], {}, {0: torch.empty(1, 1)}, {})[0], [b, c], 116)
        np.savez_compressed(f"{outdir}/u1d_sum_{tag}.npz", a=a[:1].numpy(), b=b.numpy(), c=c.numpy(), **res)

        # ---- symmetric contraction module --------------------------------------------------
        m = cuet.SymmetricContraction(O3("4x0e+4x1o+4x2e+4x3o"), O3("4x0e+4x1o"), 3, 10, layout=cue.mul_ir,
                                      dtype=dtype, original_mace=False, method="naive")
        B = 24
        x = randn(120, B, m.irreps_in.dim, dtype=dtype)
        sp = randint(121, 10, B)
        wt = randn(122, 10, *m.weight_shape, dtype=dtype) / np.sqrt(m.weight_shape[0])

        def sc_fn(w_, x_):
            m.weight.data = torch.zeros_like(m.weight.data)
            wflat = w_.flatten(1)
            return m.transpose_out(m.f([wflat, m.transpose_in(x_)], input_indices={0: sp})[0])

        res = derivatives(sc_fn, [wt, x], 123)
        np.savez_compressed(f"{outdir}/symmetric_contraction_module_{tag}.npz", weight=wt.numpy(), x=x.numpy(), species=sp.numpy(), **res)

        # ---- fully connected module ----------------------------------------------------------
        s = "4x0e+4x1o+4x2e"
        m = cuet.FullyConnectedTensorProduct(O3(s), O3(s), O3(s), layout=cue.mul_ir, internal_weights=False,
                                             shared_weights=True, method="naive")
        B = 20
        x1, x2 = randn(130, B, m.irreps_in1.dim, dtype=dtype), randn(131, B, m.irreps_in2.dim, dtype=dtype)
        wt = randn(132, 1, m.weight_numel, dtype=dtype) / 4.0
        res = derivatives(lambda w_, a_, b_: m(a_, b_, w_), [wt, x1, x2], 133)
        np.savez_compressed(f"{outdir}/fully_connected_module_{tag}.npz", weight=wt.numpy(), x1=x1.numpy(), x2=x2.numpy(), **res)

        # ---- spherical harmonics module --------------------------------------------------------
        sh = cuet.SphericalHarmonics([0, 1, 2, 3], normalize=True, method="naive")
        vec = randn(140, 32, 3, dtype=dtype)
        res = derivatives(lambda v: sh(v), [vec], 141)
        np.savez_compressed(f"{outdir}/spherical_harmonics_{tag}.npz", vec=vec.numpy(), **res)

        # ---- transpose ---------------------------------------------------------------------------
        t = cuet.TransposeIrrepsLayout(O3("3x0e+5x1o+2x2e"), source=cue.mul_ir, target=cue.ir_mul, use_fallback=True)
        x = randn(150, 6, 28, dtype=dtype)
        np.savez_compressed(f"{outdir}/transpose_{tag}.npz", x=x.numpy(), y=t(x).numpy())


if __name__ == "__main__":
    import os

    if len(sys.argv) < 2:
        raise SystemExit(f"usage: python {sys.argv[0]} <path of the cuEquivariance reference checkout>")
    main(sys.argv[1], os.path.dirname(os.path.abspath(__file__)))
