"""Helpers of the GPU parity tests: the stated float32 tolerance and its violation statistics.

Stated tolerance for float32 results: ``|a - b| <= 1e-5 |b| + 1e-6`` (relative 1e-5, absolute
1e-6).  An output entry of these operations is a sum of hundreds to thousands of O(1) products
that partly cancel, so the float32 *oracle* (same algorithm, float32 arithmetic, different
summation order) itself misses that bound against the float64 oracle.  ``report`` measures by
how much: for the CUDA result against the float32 oracle, against the float64 oracle, and for
the float32 oracle against the float64 oracle, it gives the largest and the 99.9th-percentile
value of ``|a - b| / (1e-5 |b| + 1e-6)`` (1.0 = exactly on the bound) and the fraction of
entries above 1.  The parity assertions themselves use the bound with the absolute term
scaled by the magnitude of the tensor (``close``).
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

RTOL, ATOL = 1e-5, 1e-6
ROWS: list = []


def _np(t):
    return t.detach().cpu().double().numpy() if torch.is_tensor(t) else np.asarray(t, dtype=np.float64)


def violation(a, b):
    a, b = _np(a), _np(b)
    r = np.abs(a - b) / (RTOL * np.abs(b) + ATOL)
    if r.size == 0:
        return 0.0, 0.0, 0.0
    return float(r.max()), float(np.quantile(r.reshape(-1)[:: max(1, r.size // 4_000_000)], 0.999)), float((r > 1).mean())


def report(config: str, quantity: str, got, ref32, ref64):
    """Records one row of the tolerance table (printed at the end of the session and, when
    ``CUEQ_B200_REPORT_DIR`` is set, appended to ``tolerance.jsonl`` there)."""
    row = {"config": config, "quantity": quantity, "scale": float(np.abs(_np(ref64)).max()) if _np(ref64).size else 0.0}
    for name, a, b in (("cuda_vs_f32_oracle", got, ref32), ("cuda_vs_f64_oracle", got, ref64), ("f32_oracle_vs_f64_oracle", ref32, ref64)):
        if a is None or b is None:
            continue
        mx, p999, frac = violation(a, b)
        row[name] = {"max": round(mx, 3), "p99.9": round(p999, 3), "frac_above_1": round(frac, 6)}
    ROWS.append(row)
    out_dir = os.environ.get("CUEQ_B200_REPORT_DIR")
    if out_dir:
        with open(os.path.join(out_dir, "tolerance.jsonl"), "a") as f:
            f.write(json.dumps(row) + "\n")
    print("tolerance:", json.dumps(row))
    return row


def close(a, b, rtol, atol, what=""):
    """``|a - b| <= rtol |b| + atol * max(1, max|b|)``."""
    a, b = _np(a), _np(b)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    scale = max(1.0, float(np.abs(b).max())) if b.size else 1.0
    err = np.abs(a - b) - (atol * scale + rtol * np.abs(b))
    assert np.all(err <= 0), f"{what}: max abs diff {np.abs(a - b).max():.3e} at scale {scale:.3e}, worst excess {err.max():.3e}"
