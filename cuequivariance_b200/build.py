"""Builds ``libcueq_b200.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m cuequivariance_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is rebuilt when any source under
``csrc/`` or ``include/`` is newer than the ``.so``.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libcueq_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-O3",
    "-DCUEQ_B200",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted((CSRC / "generated").glob("*.cu"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps)


def generate() -> None:
    """Regenerates csrc/generated/*.cuh (no-op when the text is unchanged)."""
    import importlib.util

    for name in ("gen_cw_groups", "gen_u1d_static", "gen_sh"):
        spec = importlib.util.spec_from_file_location(name, CSRC / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.main()


def build(force: bool = False, verbose: bool = False) -> Path:
    generate()
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    objs, procs = [], []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        if not force and obj.exists() and obj.stat().st_mtime > max(
            [src.stat().st_mtime] + [h.stat().st_mtime for h in list(CSRC.rglob("*.cuh")) + list((ROOT / "include").glob("*.h"))]
        ):
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)] + (["-Xptxas", "-v"] if verbose else [])
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
    cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("linking libcueq_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
