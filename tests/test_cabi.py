"""CPU tests of the C-ABI library: it loads, exports every symbol the header declares, and
its host-only entry points (plan creation, argument validation) behave."""
import ctypes as C
import os
import re

import pytest

import cuequivariance_b200 as cb
from cuequivariance_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "cueq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cueq_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = _declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/cueq_b200.h but not exported"
    assert L.cueq_b200_abi_version() == 1


def _desc(extent=4, bad_segment=False, math=_lib.F32):
    keep = [
        _lib.int32_array([1, 1, 0, 1]), _lib.int32_array([2, 2, 3, 2]), _lib.int32_array([4]),
        _lib.int32_array([0, 1, 2, 3]), _lib.int32_array([2]),
        _lib.int32_array([0, 0, 0, 0, 1, 1, 2, 9 if bad_segment else 1]), _lib.double_array([0.5, -2.0]),
    ]
    d = _lib.U1dDesc(extent, 3, 1, keep[0], keep[1], 1, keep[2], keep[3], keep[4], keep[5], keep[6], math)
    return d, keep


def test_plan_create_and_tables():
    L = _lib.lib()
    d, keep = _desc()
    h = C.c_void_p()
    assert L.cueq_b200_u1d_plan_create(C.byref(d), C.byref(h)) == 0
    n = L.cueq_b200_plan_table_bytes(h)
    assert n > 0 and n % 16 == 0
    assert L.cueq_b200_plan_table_data(h)
    L.cueq_b200_plan_destroy(h)


def test_plan_create_rejects_bad_input():
    L = _lib.lib()
    h = C.c_void_p()
    d, keep = _desc(bad_segment=True)
    assert L.cueq_b200_u1d_plan_create(C.byref(d), C.byref(h)) != 0
    assert b"segment" in L.cueq_b200_last_error()
    d, keep = _desc(math=_lib.BF16)
    assert L.cueq_b200_u1d_plan_create(C.byref(d), C.byref(h)) != 0
    assert b"math_dtype" in L.cueq_b200_last_error()
    d, keep = _desc(extent=0)
    assert L.cueq_b200_u1d_plan_create(C.byref(d), C.byref(h)) != 0


def test_launch_validates_arguments_before_touching_the_device():
    L = _lib.lib()
    d, keep = _desc()
    h = C.c_void_p()
    assert L.cueq_b200_u1d_plan_create(C.byref(d), C.byref(h)) == 0
    bufs = (_lib.Buffer * 4)()
    assert L.cueq_b200_u1d_launch(h, None, 4, bufs, 4, None) != 0          # no tables
    assert L.cueq_b200_u1d_launch(h, C.c_void_p(16), 4, bufs, 3, None) != 0  # wrong buffer count
    bufs[0].mode = 7
    assert L.cueq_b200_u1d_launch(h, C.c_void_p(16), 4, bufs, 4, None) != 0  # invalid mode
    assert b"mode" in L.cueq_b200_last_error()
    L.cueq_b200_plan_destroy(h)


def test_cpu_tensors_are_rejected():
    import torch

    e = cb.descriptors.channelwise_tensor_product("4x0e+4x1o", "0e+1o", ["0e", "1o"])
    m = cb.SegmentedPolynomial(e.polynomial, method="uniform_1d")
    xs = [torch.randn(3, o.size) for o in e.polynomial.inputs]
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        m(xs)


def test_method_naive_is_not_offered():
    e = cb.descriptors.linear("2x0e", "2x0e")
    with pytest.raises(ValueError, match="naive"):
        cb.SegmentedPolynomial(e.polynomial, method="naive")
    with pytest.raises(ValueError, match="uniform_1d"):
        cb.SegmentedPolynomial(cb.descriptors.fully_connected_tensor_product("2x0e+2x1o", "2x0e+2x1o", "2x0e").polynomial,
                               method="uniform_1d")


def test_lowering_matches_reference_serialisation(golden):
    """The lists handed to the kernel are the ones the reference front-end would serialise
    for the same polynomial (fixture generated from the reference's flattened tables)."""
    import numpy as np
    import torch

    from cuequivariance_b200.executor import Uniform1dProgram

    g = golden("descriptors.npz")
    e = cb.descriptors.channelwise_tensor_product("8x0e+8x1o+8x2e+8x3o", "0e+1o+2e+3o", ["0e", "1o", "2e", "3o"])
    s = Uniform1dProgram(e.polynomial, torch.float32).serialised()
    assert s["operand_extent"] == 8 and s["buffer_dim"] == [1, 1, 0, 1]
    assert s["buffer_num_segments"] == [23, 16, 16, 99]
    assert s["num_paths"] == [353]
    assert np.array_equal(np.array(s["path_indices"]).reshape(353, 4), g["cw_l3_flat/op0_indices"])
    assert np.abs(np.array(s["path_coefficients"]) - g["cw_l3_flat/op0_coefficients"]).max() < 1e-14


def test_binding_struct_sizes_match_the_library():
    L = _lib.lib()
    structs = (_lib.U1dDesc, _lib.Buffer, _lib.CwArgs, _lib.CwNoAllocArgs, _lib.GemmArgs, _lib.FctpArgs, _lib.FctpFusedArgs,
               _lib.FctpFusedTask, _lib.FctpFusedGxArgs, _lib.FctpFusedUnit, _lib.FctpFusedGwArgs, _lib.FctpFusedWUnit,
               _lib.GemmF32x3Args, _lib.GemmF32x3TnArgs, _lib.ShArgs)
    for which, st in enumerate(structs):
        assert L.cueq_b200_sizeof(which) == C.sizeof(st), st.__name__
    assert L.cueq_b200_sizeof(len(structs)) == -1


def test_tensor_core_entry_points_validate_before_launching():
    """Argument checks run on the host before any CUDA call, so they can be exercised without a GPU."""
    L = _lib.lib()
    a = _lib.FctpFusedArgs()
    assert L.cueq_b200_fctp_fused_forward(C.byref(a), None) != 0 and b"null" in L.cueq_b200_last_error()
    g = _lib.FctpFusedGxArgs()
    assert L.cueq_b200_fctp_fused_gx(C.byref(g), None) != 0 and b"null" in L.cueq_b200_last_error()
    w = _lib.FctpFusedGwArgs()
    assert L.cueq_b200_fctp_fused_gw(C.byref(w), None) != 0 and b"null" in L.cueq_b200_last_error()
    x = _lib.GemmF32x3Args()
    x.A = x.B_hi = x.B_lo = x.C = 4096
    x.M, x.N, x.K, x.lda, x.ldb, x.ldc = 128, 128, 48, 48, 48, 128
    assert L.cueq_b200_gemm_f32x3(C.byref(x), None) != 0 and b"multiple of 32" in L.cueq_b200_last_error()
    x.K = x.lda = x.ldb = 64
    x.N = 130
    assert L.cueq_b200_gemm_f32x3(C.byref(x), None) != 0 and b"multiple of 4" in L.cueq_b200_last_error()


def test_fused_fully_connected_tables():
    """Host tables of the fused fully connected kernels for 64x0e+64x1o+64x2e (11 paths):
    9 forward tasks = (output irrep, component), 23 x-gradient units (<= 2 components each),
    35 weight-gradient units = (path, component); the coupling columns they carry reproduce the
    descriptor's coefficients."""
    import numpy as np

    from cuequivariance_b200 import descriptors as D
    from cuequivariance_b200.fused_tp import DenseUVW

    s = "64x0e+64x1o+64x2e"
    e = D.fully_connected_tensor_product(s, s, s)
    dense = DenseUVW(e.polynomial, None)
    tasks, u1, u2, wu = dense._fused_tasks(), dense._fused_units(1), dense._fused_units(2), dense._fused_wunits()
    assert len(tasks) == 9 and len(u1) == 23 and len(u2) == 23 and len(wu) == 35
    assert sorted(t.num_paths for t in tasks) == [3, 4, 4, 4, 4, 4, 4, 4, 4]
    d = dense.d
    total = sum(float(np.abs(p.coefficients).sum()) for p in d.paths)
    from_tasks = sum(abs(t.paths[q].c[i]) for t in tasks for q in range(t.num_paths) for i in range(25))
    from_w = sum(abs(u.c[i]) for u in wu for i in range(25))
    from_x = sum(abs(u.c[k][i]) for u in u1 for k in range(u.nk) for i in range(25))
    for got in (from_tasks, from_w, from_x):
        assert abs(got - total) <= 1e-5 * total
    # x2 units carry the transposed coupling
    p0 = d.paths[-1]
    ua, ub = u1[-1], u2[-1]
    k = ua.nk - 1
    for i in range(p0.coefficients.shape[0]):
        for j in range(p0.coefficients.shape[1]):
            assert ua.c[k][i * 5 + j] == ub.c[k][j * 5 + i]


def test_split_tf32_halves():
    import torch

    from cuequivariance_b200.dense import split_tf32

    x = torch.randn(4096, generator=torch.Generator().manual_seed(0)) * 3
    hi, lo = split_tf32(x)
    assert int((hi.view(torch.int32) & 8191).abs().max()) == 0
    assert int((lo.view(torch.int32) & 8191).abs().max()) == 0
    assert float((hi + lo - x).abs().max()) <= 2.0 ** -21 * float(x.abs().max())
    assert float((hi - x).abs().max()) <= 2.0 ** -11 * float(x.abs().max())


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 and as C++ on its own, and a C program that
    only includes it must link against the library and read the ABI version without CUDA or torch."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    header = os.path.join(ROOT, "include", "cueq_b200.h")
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", header], check=True)
    gxx = shutil.which("g++")
    if gxx:
        subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-x", "c++", header], check=True)
    src = tmp_path / "probe.c"
    src.write_text(
        '#include <stdio.h>\n#include "cueq_b200.h"\n'
        "int main(void) {\n"
        "  cueq_gemm_f32x3_args a = {0};\n"
        '  printf("%d %lld %d\\n", cueq_b200_abi_version(), (long long)cueq_b200_sizeof(2), cueq_b200_gemm_f32x3(&a, 0) != 0);\n'
        "  return 0;\n}\n")
    exe = tmp_path / "probe"
    libdir = os.path.dirname(str(_lib.LIB_PATH))
    subprocess.run([gcc, "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe), "-L", libdir,
                    "-l:libcueq_b200.so", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert out[0] == "1" and int(out[1]) == C.sizeof(_lib.CwArgs) and out[2] == "1"


def test_product_never_touches_the_oracle_or_scratch_files():
    """The oracle is test infrastructure: nothing under the package may import or execute it, and no
    committed file may reach into the scratch directory."""
    import re

    pkg = os.path.join(ROOT, "cuequivariance_b200")
    bad = []
    for base, _dirs, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f), errors="ignore").read()
                if re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M) or "_work/" in text or "_work." in text:
                    bad.append(os.path.relpath(os.path.join(base, f), ROOT))
    assert not bad, bad
    for f in ("bench.py", "__graft_entry__.py"):
        assert "_work" not in open(os.path.join(ROOT, f)).read(), f
