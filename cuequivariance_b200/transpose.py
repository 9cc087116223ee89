"""Layout transposition modules (mul_ir <-> ir_mul).

Mirror of the reference's ``TransposeIrrepsLayout`` / ``TransposeSegments``
(cuequivariance_torch/primitives/transpose.py:23-131), executed by the CUDA
``cueq_b200_segmented_transpose`` kernel; the transposition is its own adjoint up to
swapping the tile shape, which gives the backward.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.nn as nn

from . import _lib
from .executor import dtype_code
from .irreps import Irreps, IrrepsLayout


def _launch(x: torch.Tensor, info: torch.Tensor) -> torch.Tensor:
    if x.device.type != "cuda":
        raise RuntimeError("cuequivariance_b200 executes on CUDA devices only (there is no CPU fallback)")
    x = x.contiguous()
    y = torch.empty_like(x)
    rows = x.shape[0] if x.ndim > 1 else 1
    flat_rows = x.numel() // x.shape[-1] if x.shape[-1] else 0
    with torch.cuda.device(x.device):
        _lib.check(
            _lib.lib().cueq_b200_segmented_transpose(
                x.data_ptr(), y.data_ptr(), flat_rows, x.shape[-1], info.data_ptr(), info.shape[0],
                dtype_code(x.dtype), C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream),
            )
        )
    del rows
    return y


class _TransposeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, info_fwd, info_bwd):
        ctx.info = (info_fwd, info_bwd)
        return _launch(x, info_fwd)

    @staticmethod
    def backward(ctx, g):
        info_fwd, info_bwd = ctx.info
        return _TransposeFn.apply(g, info_bwd, info_fwd), None, None


class TransposeSegments(nn.Module):
    """``segments``: list of ``(u, v)``; each [u, v] tile of a row becomes [v, u]."""

    def __init__(self, segments, device: Optional[torch.device] = None):
        super().__init__()
        fwd, bwd, off = [], [], 0
        for u, v in segments:
            if u > 1 and v > 1:
                fwd.append([off, u, v, -1])
                bwd.append([off, v, u, -1])
            off += u * v
        self.dim = off
        self.trivial = len(fwd) == 0
        # blocks that are left alone still have to be copied: describe them as [1, n] tiles
        full_f, full_b, off = [], [], 0
        for u, v in segments:
            if u > 1 and v > 1:
                full_f.append([off, u, v, -1])
                full_b.append([off, v, u, -1])
            else:
                full_f.append([off, 1, u * v, -1])
                full_b.append([off, 1, u * v, -1])
            off += u * v
        self.register_buffer("info_fwd", torch.tensor(full_f, dtype=torch.int32, device=device).reshape(-1, 4), persistent=False)
        self.register_buffer("info_bwd", torch.tensor(full_b, dtype=torch.int32, device=device).reshape(-1, 4), persistent=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.trivial:
            return x
        if self.info_fwd.device != x.device:
            self.info_fwd = self.info_fwd.to(x.device)
            self.info_bwd = self.info_bwd.to(x.device)
        return _TransposeFn.apply(x, self.info_fwd, self.info_bwd)


class TransposeIrrepsLayout(nn.Module):
    """Changes the layout of a tensor of irreps; identity when source == target."""

    def __init__(self, irreps, *, source, target, device: Optional[torch.device] = None, use_fallback: Optional[bool] = None):
        super().__init__()
        irreps = irreps if isinstance(irreps, Irreps) else Irreps(irreps)
        source, target = IrrepsLayout.parse(source), IrrepsLayout.parse(target)
        self.irreps, self.source, self.target = irreps, source, target
        if source is target:
            self.f = None
        elif source is IrrepsLayout.mul_ir:
            self.f = TransposeSegments([(mul, ir.dim) for mul, ir in irreps], device)
        else:
            self.f = TransposeSegments([(ir.dim, mul) for mul, ir in irreps], device)

    def extra_repr(self) -> str:
        return f"{self.source.name} -> {self.target.name}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x if self.f is None else self.f(x)


_INFO_CACHE: dict = {}


def transpose_blocks(x: torch.Tensor, blocks, to_ir_mul: bool) -> torch.Tensor:
    """Explicit layout change of a row-major ``[rows, sum(mul*dim)]`` tensor (no autograd):
    ``blocks`` = ((mul, dim), ...); mul_ir -> ir_mul when ``to_ir_mul`` else the reverse."""
    key = (tuple(blocks), bool(to_ir_mul), x.device)
    info = _INFO_CACHE.get(key)
    if info is None:
        rows, off = [], 0
        for mul, dim in blocks:
            u, v = (mul, dim) if to_ir_mul else (dim, mul)
            rows.append([off, u, v, -1] if (u > 1 and v > 1) else [off, 1, u * v, -1])
            off += mul * dim
        info = torch.tensor(rows, dtype=torch.int32, device=x.device).reshape(-1, 4)
        _INFO_CACHE[key] = info
    return _launch(x, info)
