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
