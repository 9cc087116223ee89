"""TEST INFRASTRUCTURE ONLY - the CPU oracle streamed over the batch axis.

The naive evaluation (``oracle/naive.py``, restating
cuequivariance_torch/primitives/segmented_polynomial_naive.py:61-246,308-435) materialises
every per-path product for the whole batch: about 0.33 MB of host memory per edge for the
128-channel, lmax-3 channelwise product.  Outputs that are scatter-added (or summed) over
the batch are sums of per-row terms, so the batch can be cut into chunks that are
evaluated one after the other and accumulated; in float64 that is exact up to the order
of additions, and every derivative of a scalar that is itself a sum over the batch
decomposes the same way.  Two runners:

* ``forward``: outputs of a polynomial, chunk by chunk;
* ``value_and_grads``: a scalar objective ``sum_chunks f(chunk)`` with gradients, where the
  gradients of per-row operands are concatenated and those of shared / gathered operands
  are accumulated.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch

from . import naive


def forward(poly, inputs: Sequence[torch.Tensor], input_indices: Optional[Dict[int, torch.Tensor]], output_rows: Dict[int, int],
            output_indices: Dict[int, torch.Tensor], batch: int, chunk: int = 4096, accumulate_dtype=torch.float64,
            math_dtype=None) -> List[torch.Tensor]:
    """Every output must be scatter-added through ``output_indices`` (accumulated over the
    chunks in ``accumulate_dtype``).  Inputs with ``batch`` rows and all index tensors are
    cut along the batch; gathered and shared inputs are passed whole."""
    input_indices = dict(input_indices or {})
    outs = {j: torch.zeros(rows, poly.outputs[j].size, dtype=accumulate_dtype) for j, rows in output_rows.items()}
    assert set(outs) == set(range(len(poly.outputs))) == set(output_indices)
    for a in range(0, batch, chunk):
        b = min(batch, a + chunk)
        xs = [x[a:b] if (k not in input_indices and x.shape[0] == batch) else x for k, x in enumerate(inputs)]
        ii = {k: v[a:b] for k, v in input_indices.items()}
        oi = {k: v[a:b] for k, v in output_indices.items()}
        res = naive.segmented_polynomial(poly, xs, ii, output_rows, oi, math_dtype=math_dtype)
        for j, r in enumerate(res):
            outs[j] += r.to(accumulate_dtype)
    return [outs[j] for j in range(len(poly.outputs))]


def value_and_grads(fn: Callable[[Sequence[torch.Tensor], Sequence[torch.Tensor]], torch.Tensor],
                    per_row: Sequence[torch.Tensor], whole: Sequence[torch.Tensor], batch: int, chunk: int = 4096,
                    accumulate_dtype=torch.float64, extra: Optional[Callable] = None):
    """``fn(per_row_chunk, whole) -> scalar`` contribution of one chunk (``per_row_chunk`` are
    the rows ``a:b`` of every tensor in ``per_row``, with ``requires_grad`` set; index tensors
    can be passed among them, integer tensors get no gradient).  Returns the total, the
    gradients of the per-row tensors (concatenated; None for integer tensors) and the
    gradients of the ``whole`` tensors (accumulated).  ``extra(per_row_chunk, whole)``, when
    given, is called inside the same graph and must return a list of tensors with one row per
    batch row; they are concatenated and returned as a fourth value (used for intermediate
    quantities such as first derivatives)."""
    total = torch.zeros((), dtype=accumulate_dtype)
    g_whole = [torch.zeros(t.shape, dtype=accumulate_dtype) for t in whole]
    g_rows: List[List[torch.Tensor]] = [[] for _ in per_row]
    extras: List[List[torch.Tensor]] = []
    for a in range(0, batch, chunk):
        b = min(batch, a + chunk)
        rows = [t[a:b].clone().requires_grad_(True) if t.is_floating_point() else t[a:b] for t in per_row]
        ws = [t.clone().requires_grad_(True) for t in whole]
        val = fn(rows, ws)
        if extra is not None:
            ex = extra(rows, ws)
            if not extras:
                extras = [[] for _ in ex]
            for lst, t in zip(extras, ex):
                lst.append(t.detach())
        diff = [t for t in rows if t.is_floating_point()] + ws
        gs = torch.autograd.grad(val, diff, allow_unused=True)
        total += val.detach().to(accumulate_dtype)
        it = iter(gs)
        for k, t in enumerate(rows):
            if t.is_floating_point():
                g = next(it)
                g_rows[k].append(torch.zeros_like(t) if g is None else g)
        for k in range(len(ws)):
            g = next(it)
            if g is not None:
                g_whole[k] += g.to(accumulate_dtype)
    rows_out = [torch.cat(lst) if lst else None for lst in g_rows]
    res = (total, rows_out, g_whole)
    return res + ([torch.cat(lst) for lst in extras],) if extra is not None else res
