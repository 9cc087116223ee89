"""pytest plugin (``-p ref_pytest_plugin`` with ``baseline/`` on PYTHONPATH): before any test
module is imported, makes the staged reference importable and installs this library's
stand-in for the closed kernel package, so the reference's own tests exercise the CUDA
kernels of this repository through the reference front-end."""
import refenv

refenv.activate(with_kernels=True)
