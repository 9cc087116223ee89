"""CPU tests of the host-side logic around the kernels: the channelwise plan built from the descriptor,
the CSR over receivers (also in sender-range passes), and the registration of the build-time straight-line
kernels."""
import numpy as np
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import _lib, descriptors as D
from cuequivariance_b200 import channelwise as cw
from cuequivariance_b200 import static_poly


def _cfg3():
    return D.channelwise_tensor_product("128x0e+128x1o+128x2e+128x3o", "0e+1o+2e+3o", ["0e", "1o", "2e", "3o"])


def test_channelwise_plan_for_the_headline_configuration():
    """Config 3: four launches (one per irrep of x1), 23 paths in total, every path's weight and output
    segment used once, 353 coupling terms compacted into 311 (i, k) pairs, blocks adjacent in the row."""
    e = _cfg3()
    plan = cw.match_channelwise(e.polynomial)
    assert plan is not None and plan.extent == 128
    assert plan.row_sizes == (2944, 2048, 16, 12672)
    assert [g["l1"] for g in plan.groups] == [0, 1, 2, 3]
    assert sum(g["npath"] for g in plan.groups) == 23
    assert [g["x1_off"] for g in plan.groups] == [0, 128, 512, 1152]
    assert [g["x1_width"] for g in plan.groups] == [128, 384, 640, 896]
    w_offs = sorted(o for g in plan.groups for o in g["w_off"])
    assert w_offs == [128 * i for i in range(23)]
    out_offs = sorted(o for g in plan.groups for o in g["out_off"])
    assert len(set(out_offs)) == 23 and out_offs[0] == 0
    assert sum(g["nterm"] for g in plan.groups) == 353
    assert sum(len(g["bwd_tab"][0]) - 1 for g in plan.groups) == 311          # non-zero (i, k) pairs (backward table)
    assert sum(len(g["fwd_tab"][0]) - 1 for g in plan.groups) == 207          # distinct values among them (forward table)
    for g in plan.groups:   # every backward entry is plus or minus one forward entry
        fwd = {tuple(sorted(zip(g["fwd_tab"][1][a:b], np.round(g["fwd_tab"][2][a:b], 12)))) for a, b in zip(g["fwd_tab"][0][:-1], g["fwd_tab"][0][1:])}
        for a, b in zip(g["bwd_tab"][0][:-1], g["bwd_tab"][0][1:]):
            terms = sorted(zip(g["bwd_tab"][1][a:b], np.round(g["bwd_tab"][2][a:b], 12)))
            neg = sorted((j, -c) for j, c in terms)
            assert tuple(terms) in fwd or tuple(neg) in fwd
    lib = cw._library_groups()
    assert all(0 <= g["id"] < _lib.lib().cueq_b200_cw_num_groups() for g in plan.groups) and len(lib) >= 4


def test_channelwise_plan_rejects_other_polynomials():
    e = D.fully_connected_tensor_product("4x0e+4x1o", "4x0e+4x1o", "4x0e+4x1o")
    assert cw.match_channelwise(e.polynomial) is None
    e = D.channelwise_tensor_product("8x0e+8x1o", "0e+1o+2e+3o+4e", ["0e", "1o", "2e", "3o", "4e"])   # l = 4 has no built-in group
    assert cw.match_channelwise(e.polynomial) is None


def test_csr_over_receivers():
    gen = torch.Generator().manual_seed(3)
    n_rows, n_edges = 17, 200
    idx = torch.randint(0, n_rows, (n_edges,), generator=gen, dtype=torch.int32)
    cache = cw._CsrCache()
    order, rowptr = cache.get(idx, n_rows)
    assert order is not None and rowptr.shape == (n_rows + 1,) and int(rowptr[-1]) == n_edges
    sorted_idx = idx[order.long()]
    assert bool((sorted_idx[1:] >= sorted_idx[:-1]).all())
    counts = torch.bincount(idx.long(), minlength=n_rows)
    assert torch.equal((rowptr[1:] - rowptr[:-1]).long(), counts)
    assert cache.get(idx, n_rows)[1] is rowptr                      # cached on the tensor's identity and version
    idx[0] = (idx[0] + 1) % n_rows                                  # in-place change bumps the version
    assert cache.get(idx, n_rows)[1] is not rowptr
    s = torch.sort(idx).values
    order2, rowptr2 = cache.get(s, n_rows)
    assert order2 is None and int(rowptr2[-1]) == n_edges           # already sorted: no permutation


def test_csr_in_sender_range_passes():
    gen = torch.Generator().manual_seed(4)
    n_rows, n_send, n_edges, passes = 11, 40, 300, 2
    rcv = torch.sort(torch.randint(0, n_rows, (n_edges,), generator=gen, dtype=torch.int32)).values
    snd = torch.randint(0, n_send, (n_edges,), generator=gen, dtype=torch.int32)
    order, rowptr = cw._CsrCache().get_passes(rcv, snd, n_rows, n_send, passes)
    assert rowptr.shape == (passes * n_rows + 1,) and int(rowptr[-1]) == n_edges
    span = (n_send + passes - 1) // passes
    for row in range(passes * n_rows):
        edges = order[int(rowptr[row]) : int(rowptr[row + 1])].long()
        assert bool((rcv[edges] == row % n_rows).all())
        assert bool(((snd[edges] // span) == row // n_rows).all())
    assert sorted(order.tolist()) == list(range(n_edges))


def test_static_kernels_are_registered_for_config_1():
    """The symmetric contraction of config 1 (forward and the two merged backward programs) must find its
    build-time kernel by digest; a different polynomial must not."""
    L = _lib.lib()
    names = []
    for name, poly in static_poly.registered_polynomials():
        dg = static_poly.digest(poly)
        assert len(dg) == 16
        idx = L.cueq_b200_u1d_static_find(dg.encode())
        assert idx >= 0, name
        names.append(L.cueq_b200_u1d_static_name(idx).decode())
    assert len(names) >= 2 and len(set(names)) == len(names)
    other = D.channelwise_tensor_product("4x0e+4x1o", "0e+1o", ["0e", "1o"]).polynomial.flatten_coefficient_modes().squeeze_modes()
    assert L.cueq_b200_u1d_static_find(static_poly.digest(other).encode()) < 0


def test_merged_symmetric_paths_counts():
    """Path counts of config 1 after merging symmetric duplicates (forward 4 / 51 / 425; backward with respect to
    the weights 4 / 51 / 425, with respect to the features 4 / 86 / 1072): the numbers the reference reports for
    its unsymmetrised polynomials."""
    m = cb.SymmetricContraction("128x0e+128x1o+128x2e+128x3o", "128x0e+128x1o", 3, 10, layout=cb.mul_ir)
    fwd = static_poly.merge_symmetric_paths(m.f.polynomial)
    assert sorted(len(d.paths) for _, d in fwd.operations) == [4, 51, 425]
    bwd = m.f.polynomial.backward([True, True], [True])
    merged = static_poly.merge_symmetric_paths(bwd)
    assert sorted(len(d.paths) for _, d in merged.operations) == [4, 4, 51, 86, 425, 1072]


def test_fused_tp_flattening_choices():
    """`uv,iu,iv` with equal multiplicities keeps v as the channel axis (one path per (irrep, i, u)); with mixed
    small multiplicities every mode is flattened; with mixed large ones only the dense route remains."""
    from cuequivariance_b200.fused_tp import FusedTPProgram

    e = D.linear("8x0e+8x1o", "8x0e+8x1o")
    prog = FusedTPProgram(e.polynomial, torch.float32)
    assert prog.extent == 8 and sum(len(d.paths) for _, d in prog.flat.operations) == 8 * (1 + 3)
    e = D.linear("6x0e+5x1o", "3x0e+7x1o")
    prog = FusedTPProgram(e.polynomial, torch.float32)
    assert prog.extent == 1 and sum(len(d.paths) for _, d in prog.flat.operations) == 6 * 3 + 3 * 5 * 7
    m = cb.Linear("128x0e+128x1o", "64x0e+96x1o", layout=cb.ir_mul)
    assert m.f is None and m._dense_plan is not None and len(m._dense_plan["paths"]) == 2
    try:
        m(torch.zeros(4, m.irreps_in.dim))
    except ValueError as err:
        assert "dense route" in str(err)
    else:
        raise AssertionError("a CPU tensor must not be accepted")


def test_module_argument_errors():
    """Same error behaviour as the reference modules for inconsistent weight arguments; CPU tensors raise."""
    import pytest

    m = cb.Linear("4x0e+4x1o", "4x0e+4x1o", layout=cb.ir_mul, weight_classes=3)
    assert m.weight.shape == (3, m.weight_numel)
    with pytest.raises(ValueError, match="weight_indices"):
        m(torch.zeros(2, m.irreps_in.dim))
    with pytest.raises(ValueError, match="Internal weights"):
        m(torch.zeros(2, m.irreps_in.dim), torch.zeros(3, m.weight_numel), weight_indices=torch.zeros(2, dtype=torch.int64))
    with pytest.raises(ValueError, match="shared"):
        cb.Linear("4x0e", "4x0e", layout=cb.ir_mul, shared_weights=False, internal_weights=True)
    tp = cb.ChannelWiseTensorProduct("4x0e+4x1o", "0e+1o", ["0e", "1o"], layout=cb.mul_ir, shared_weights=False, internal_weights=False)
    with pytest.raises(RuntimeError, match="CUDA"):
        tp(torch.zeros(3, tp.irreps_in1.dim), torch.zeros(3, tp.irreps_in2.dim), torch.zeros(3, tp.weight_numel))
    from cuequivariance_b200.dense import gemm_f32x3, gemm_f32x3_tn, linear_f32x3

    for fn, args in ((gemm_f32x3, (torch.zeros(4, 32), torch.zeros(8, 32))), (gemm_f32x3_tn, (torch.zeros(4, 8), torch.zeros(4, 8))),
                     (linear_f32x3, (torch.zeros(4, 32), torch.zeros(8, 32)))):
        with pytest.raises(RuntimeError, match="CUDA"):
            fn(*args)
