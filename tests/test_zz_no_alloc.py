"""GPU test of `cueq_b200_cw_forward_noalloc`, the forward entry point for callers that are
not allowed to allocate device memory (plugin hosts that pass only input/output buffers,
code running under a foreign allocator, loops where cudaMalloc is banned).  It keeps the
CSR row pointers and the term tables in an array built into the library instead of taking
them from the caller.  The test drives it through the C ABI with buffers allocated by the
test itself, twice in a row with different graphs (the second call reuses the same built-in
array), and compares with the regular entry point, which runs the same arithmetic: the
results must agree to the float32 tolerance of the other channelwise tests (in practice
they are bit-identical).  Collected last on purpose.
"""
import ctypes as C

import pytest
import torch

import cuequivariance_b200 as cb
from cuequivariance_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_noalloc(plan, layout_mul_ir, w, x1, x2, senders, receivers, n_recv):
    L = _lib.lib()
    out = torch.full((n_recv, plan.row_sizes[3]), float("nan"), dtype=torch.float32, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for g in plan.groups:
        start, tj, tc = g["fwd_tab"]
        a = _lib.CwNoAllocArgs()
        a.w, a.x1, a.x2, a.out = w.data_ptr(), x1.data_ptr(), x2.data_ptr(), out.data_ptr()
        a.senders, a.receivers = senders.data_ptr(), receivers.data_ptr()
        keep = ((C.c_int32 * len(start))(*start), (C.c_int32 * len(tj))(*tj), (C.c_float * len(tc))(*tc))
        a.tab_start_host, a.tab_j_host, a.tab_c_host = keep
        a.w_stride, a.x1_stride, a.x2_stride, a.out_stride = plan.row_sizes
        a.num_edges, a.num_receivers = receivers.numel(), n_recv
        a.extent, a.x1_offset, a.num_paths, a.num_terms = plan.extent, g["x1_off"], g["npath"], g["nterm_fwd"]
        for q in range(g["npath"]):
            a.w_offset[q], a.out_offset[q] = g["w_off"][q], g["out_off"][q]
        a.mul_ir = 1 if layout_mul_ir else 0
        _lib.check(L.cueq_b200_cw_forward_noalloc(g["id"], C.byref(a), stream))
    return out


@pytest.mark.parametrize("mul_ir", [True, False])
def test_noalloc_forward_matches_regular_entry_point_twice(mul_ir):
    s1 = "64x0e+64x1o+64x2e+64x3o"
    tp = cb.ChannelWiseTensorProduct(s1, "0e+1o+2e+3o", ["0e", "1o", "2e", "3o"], layout=cb.mul_ir if mul_ir else cb.ir_mul,
                                     shared_weights=False, internal_weights=False)
    plan = tp.f._program(torch.float32)._special.plan
    gen = torch.Generator(device=DEV).manual_seed(7)
    for E, N in ((700, 90), (333, 41)):          # two calls in a row, different graphs
        x1 = torch.randn(N, tp.irreps_in1.dim, generator=gen, device=DEV)
        x2 = torch.randn(E, 16, generator=gen, device=DEV)
        w = torch.randn(E, tp.weight_numel, generator=gen, device=DEV)
        snd = torch.randint(0, N, (E,), generator=gen, device=DEV, dtype=torch.int32)
        rcv = torch.sort(torch.randint(0, N - 3, (E,), generator=gen, device=DEV, dtype=torch.int32)).values
        ref = tp(x1, x2, w, indices_1=snd, indices_out=rcv, size_out=N)
        got = _run_noalloc(plan, mul_ir, w, x1, x2, snd, rcv, N)
        torch.cuda.synchronize()
        assert not torch.isnan(got).any(), "some output rows were not written"
        scale = max(1.0, float(ref.abs().max()))
        assert bool(((got - ref).abs() <= 1e-5 * ref.abs() + 2e-6 * scale).all())


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    L = _lib.lib()
    a = _lib.CwNoAllocArgs()
    a.num_receivers = 262144 + 1
    assert L.cueq_b200_cw_forward_noalloc(0, C.byref(a), None) != 0
    assert b"exceed" in L.cueq_b200_last_error()
