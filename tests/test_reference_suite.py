"""The reference's own torch tests, unmodified, run against this library through the import
boundary of the closed kernel package (``cuequivariance_ops_torch`` stand-in in
``cuequivariance_b200/compat``): the reference front-end packs its argument lists, the
registered op / the ``FusedTensorProductOp`` classes of the stand-in hand them to the CUDA
kernels, and the tests compare with the reference's ``naive`` method themselves
(cuequivariance_torch/tests/primitives/segmented_polynomial_test.py:208-265: every
shared / indexed / batched combination, first derivatives and double backward;
tests/operations/channel_wise_test.py:231-305: fused gather/scatter equals explicit gather,
product and scatter_add, with double backward).

The reference is staged under ``baseline/_ref`` by ``baseline/stage_reference.py`` (it is not
part of this repository's history); the tests are skipped when it is missing.  They run in a
child process so that the reference import does not leak into the other tests.  Left out:
the export modes (TorchScript, torch.export, ONNX, TensorRT), which need the closed package's
native operator registrations, and the triangle / attention tests.
"""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASELINE = os.path.join(ROOT, "baseline")
TESTS = os.path.join(BASELINE, "_ref", "reference_tests")

SELECTIONS = [
    ("primitives/segmented_polynomial_test.py", "test_segmented_polynomial_indexing"),
    # device1 = CPU tensors handed to the closed op; this library has no CPU path by design
    ("primitives/segmented_polynomial_test.py", "test_segmented_polynomial_dytpes and not device1"),
    ("operations/channel_wise_test.py", "test_channel_wise_fwd or test_channel_wise_bwd_bwd or test_channel_wise_indexing"),
    ("operations/fully_connected_test.py", "test_fully_connected"),
    ("primitives/segmented_polynomial_test.py", "test_segmented_polynomial_indexed_linear"),
    ("operations/linear_test.py", "test_linear_fwd or test_linear_bwd_bwd or test_linear_copy"),
    ("operations/rotation_test.py", "test_rotation or test_inversion"),   # test_vector_to_euler_angles uses CPU tensors
    ("operations/spherical_harmonics_test.py", "not export"),
    ("primitives/transpose_test.py", "test_transpose"),
]


@pytest.mark.gpu
@pytest.mark.parametrize("path,select", SELECTIONS, ids=[f"{p.split('/')[-1]}::{s.split(' ')[0]}" for p, s in SELECTIONS])
def test_reference_tests_pass_on_this_library(path, select):
    if not os.path.isdir(TESTS):
        pytest.skip("the reference is not staged under baseline/_ref")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([BASELINE, ROOT, env.get("PYTHONPATH", "")])
    cmd = [sys.executable, "-m", "pytest", "-p", "ref_pytest_plugin", "-q", "-x", "--no-header", "-p", "no:cacheprovider",
           "--rootdir", TESTS, os.path.join(TESTS, path), "-k", select]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env, cwd=TESTS)
    tail = "\n".join((r.stdout + r.stderr).splitlines()[-40:])
    out_dir = os.environ.get("CUEQ_B200_REPORT_DIR")
    if out_dir and r.returncode != 0:
        with open(os.path.join(out_dir, "reference_suite_failure_" + os.path.basename(path) + ".log"), "w") as f:
            f.write(r.stdout + r.stderr)
    assert r.returncode == 0, tail
    m = re.search(r"(\d+) passed", r.stdout)
    assert m and int(m.group(1)) > 0, "no reference test ran:\n" + tail
    if out_dir:
        with open(os.path.join(out_dir, "reference_suite.txt"), "a") as f:
            f.write(f"{path} -k '{select}': {r.stdout.strip().splitlines()[-1]}\n")
