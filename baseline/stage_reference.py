"""Stages the unmodified reference (NVIDIA/cuEquivariance, pure Python) under ``baseline/_ref``.

    python baseline/stage_reference.py [path to the reference checkout]

``baseline/_ref`` is ignored by git but travels with the working tree to the machine that has
the GPU, where the reference checkout itself does not exist.  What is staged there is used as
the *checker* and as the timed CPU baseline only (``tests/``, ``bench.py --impl reference``,
the ``cpu_baseline`` leg); nothing in the ``cuequivariance_b200`` package imports it.

The regular route, ``pip install --no-index --no-build-isolation --target baseline/_ref
<checkout>/cuequivariance``, stops at the build backend (``hatchling`` is not installed and
cannot be fetched), so the script does what installing those two pure-Python wheels would do:
it copies the package directories ``cuequivariance`` and ``cuequivariance_torch`` (with the
``VERSION`` file they read through a symlink) and, next to them, the reference's own torch
test-suite, which the GPU tests run unmodified against this library's stand-in for the closed
kernel package.  The outcome of the pip attempt is written to ``baseline/_ref/STAGED.txt``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def default_checkout() -> str:
    return os.environ.get("CUEQ_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def stage(checkout: str | None = None, try_pip: bool = False) -> bool:
    """Returns True when ``baseline/_ref`` holds the reference afterwards."""
    checkout = checkout or default_checkout()
    if not os.path.isdir(os.path.join(checkout, "cuequivariance", "cuequivariance")):
        return os.path.isdir(os.path.join(DEST, "cuequivariance"))
    note = "pip install not attempted"
    if try_pip:
        r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--find-links",
                            "/opt/wheelhouse", "--target", os.path.join(DEST, "_pip"), os.path.join(checkout, "cuequivariance")],
                           capture_output=True, text=True)
        note = "pip install exit code %d: %s" % (r.returncode, (r.stderr.strip().splitlines() or ["ok"])[-1])
        shutil.rmtree(os.path.join(DEST, "_pip"), ignore_errors=True)
    os.makedirs(DEST, exist_ok=True)
    version = open(os.path.join(checkout, "VERSION")).read()
    for pkg in ("cuequivariance", "cuequivariance_torch"):
        dst = os.path.join(DEST, pkg)
        shutil.rmtree(dst, ignore_errors=True)
        shutil.copytree(os.path.join(checkout, pkg, pkg), dst, symlinks=False,
                        ignore=shutil.ignore_patterns("__pycache__", "VERSION", "SKILL.md"))
        with open(os.path.join(dst, "VERSION"), "w") as f:
            f.write(version)
    tests = os.path.join(DEST, "reference_tests")
    shutil.rmtree(tests, ignore_errors=True)
    shutil.copytree(os.path.join(checkout, "cuequivariance_torch", "tests"), tests, ignore=shutil.ignore_patterns("__pycache__"))
    for root, _, files in os.walk(DEST):      # the checkout is read-only; the copy must be removable
        os.chmod(root, 0o755)
        for f in files:
            os.chmod(os.path.join(root, f), 0o644)
    with open(os.path.join(DEST, "STAGED.txt"), "w") as f:
        f.write(f"reference version {version.strip()} copied from {checkout}\n{note}\n")
    return True


if __name__ == "__main__":
    ok = stage(sys.argv[1] if len(sys.argv) > 1 else None, try_pip=True)
    print("staged" if ok else "reference checkout not found; nothing staged", DEST)
