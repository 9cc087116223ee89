"""float32-accurate dense layer on the tensor cores (three TF32 passes).

``linear_f32x3(x, weight, bias)`` computes ``x @ weight.T + bias`` like ``torch.nn.functional.linear``
for float32 CUDA tensors whose number of input features is a multiple of 32.  It is meant for the layer that produces
the per-edge weights of a channelwise tensor product from a few edge scalars (the pattern of the
reference's convolution layer, cuequivariance_torch/layers/tp_conv_fully_connected.py:145-152,219-238):
at 1M edges x 2,944 weights that layer is 0.39 TFLOP, an order of magnitude more time than the
tensor product itself when it runs on the CUDA cores.

Forward, input gradient, weight gradient and bias gradient all run on this library's tcgen05 kernels
(``csrc/gemm_f32x3.cu``: one that keeps the split A tile resident for K <= 64, one that streams both
operands for larger K, one that reduces over rows and transposes the blocks in shared memory).
"""
from __future__ import annotations

from typing import Optional

import torch


def split_tf32(x: torch.Tensor):
    """``x = hi + lo`` (up to 2^-21 relative) with both halves exactly representable in TF32:
    the low 13 mantissa bits of each are zero (round to nearest, ties away from zero)."""
    def rna(t):  # round to 10 mantissa bits, ties away from zero (what cvt.rna.tf32.f32 does)
        return ((t.contiguous().view(torch.int32) + 4096) & -8192).view(torch.float32)

    hi = rna(x)
    lo = rna(x - hi)
    return hi, lo


def _rows_view_ok(t: torch.Tensor) -> bool:
    return t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 4 == 0 and t.data_ptr() % 16 == 0


def gemm_f32x3(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, name: str = "gemm_f32x3",
               out: Optional[torch.Tensor] = None, b_split=None) -> torch.Tensor:
    """``a [M, K] @ b[N, K].T (+ bias[N])`` in float32 accuracy on the tensor cores; K a multiple of 32,
    N a multiple of 4.  ``a`` and ``out`` may be column slices of wider row-major tensors (unit stride
    along the row, 16-byte aligned); ``out`` is overwritten.  ``b_split = split_tf32(b)`` may be passed by a
    caller that multiplies by the same ``b`` several times."""
    import ctypes as C

    from . import _lib, profiling

    if not (a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32):
        raise RuntimeError("gemm_f32x3 needs float32 CUDA tensors (there is no CPU fallback)")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1] or a.shape[1] % 32 or a.shape[1] == 0:
        raise ValueError(f"gemm_f32x3: a [M, K] and b [N, K] with K a multiple of 32; got {tuple(a.shape)}, {tuple(b.shape)}")
    if b.shape[0] % 4:
        raise ValueError("gemm_f32x3: the number of output columns must be a multiple of 4")
    ac = a if _rows_view_ok(a) else a.contiguous()
    hi, lo = b_split if b_split is not None else split_tf32(b)
    if out is None:
        out = torch.empty((a.shape[0], b.shape[0]), dtype=torch.float32, device=a.device)
    elif not (_rows_view_ok(out) and out.shape == (a.shape[0], b.shape[0]) and out.dtype == torch.float32):
        raise ValueError("gemm_f32x3: `out` must be a float32 [M, N] view with unit stride along rows and 16-byte alignment")
    if a.shape[0] == 0:
        return out
    status = _lib.status_word(a.device)
    g = _lib.GemmF32x3Args()
    g.A, g.B_hi, g.B_lo, g.C = ac.data_ptr(), hi.data_ptr(), lo.data_ptr(), out.data_ptr()
    bc = None
    if bias is not None:
        bc = bias.contiguous()
        g.bias = bc.data_ptr()
    g.M, g.N, g.K = ac.shape[0], b.shape[0], ac.shape[1]
    g.lda, g.ldb, g.ldc = ac.stride(0), hi.shape[1], out.stride(0)
    g.status = status.data_ptr()
    with torch.cuda.device(a.device):
        with profiling.kernel(name):
            _lib.check(_lib.lib().cueq_b200_gemm_f32x3(C.byref(g), C.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)))
    return out


def gemm_f32x3_tn(a: torch.Tensor, b: torch.Tensor, with_colsum: bool = False, name: str = "gemm_f32x3_tn",
                  out: Optional[torch.Tensor] = None):
    """``a[K, M].T @ b[K, N]`` (and, with ``with_colsum``, ``a.sum(0)``) in float32 accuracy on the tensor
    cores: the reduction runs over the rows of both operands.  M and N multiples of 4; ``a`` and ``b`` may
    be column slices of wider row-major tensors.  ``out`` (float32 [M, N], contiguous rows) is ADDED to."""
    import ctypes as C

    from . import _lib, profiling

    if not (a.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32):
        raise RuntimeError("gemm_f32x3_tn needs float32 CUDA tensors (there is no CPU fallback)")
    if a.dim() != 2 or b.dim() != 2 or a.shape[0] != b.shape[0] or a.shape[1] % 4 or b.shape[1] % 4:
        raise ValueError(f"gemm_f32x3_tn: a [K, M] and b [K, N] with M, N multiples of 4; got {tuple(a.shape)}, {tuple(b.shape)}")
    ac = a if _rows_view_ok(a) else a.contiguous()
    bc = b if _rows_view_ok(b) else b.contiguous()
    if out is None:
        out = torch.zeros((a.shape[1], b.shape[1]), dtype=torch.float32, device=a.device)
    elif not (_rows_view_ok(out) and out.shape == (a.shape[1], b.shape[1]) and out.dtype == torch.float32):
        raise ValueError("gemm_f32x3_tn: `out` must be a float32 [M, N] view with unit stride along rows and 16-byte alignment")
    colsum = torch.zeros(a.shape[1], dtype=torch.float32, device=a.device) if with_colsum else None
    if a.shape[0] > 0:
        status = _lib.status_word(a.device)
        g = _lib.GemmF32x3TnArgs()
        g.A, g.B, g.C = ac.data_ptr(), bc.data_ptr(), out.data_ptr()
        if colsum is not None:
            g.colsum = colsum.data_ptr()
        g.M, g.N, g.K = a.shape[1], b.shape[1], a.shape[0]
        g.lda, g.ldb, g.ldc = ac.stride(0), bc.stride(0), out.stride(0)
        g.status = status.data_ptr()
        with torch.cuda.device(a.device):
            with profiling.kernel(name):
                _lib.check(_lib.lib().cueq_b200_gemm_f32x3_tn(C.byref(g), C.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)))
    return (out, colsum) if with_colsum else out


class _LinearF32x3(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        out = gemm_f32x3(x, weight.detach(), bias.detach() if bias is not None else None)
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return out

    @staticmethod
    def backward(ctx, gout):
        x, weight = ctx.saved_tensors
        gout = gout.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            if weight.shape[0] % 32 == 0 and weight.shape[1] % 4 == 0:
                gx = gemm_f32x3(gout, weight.detach().t().contiguous(), name="gemm_f32x3_gx")   # gout [M, N] x (W^T [K, N])^T
            else:
                gx = _full_precision_matmul(gout, weight)
        gb = None
        want_gb = ctx.has_bias and ctx.needs_input_grad[2]
        if ctx.needs_input_grad[1] and gout.shape[1] % 4 == 0 and x.shape[1] % 4 == 0:
            res = gemm_f32x3_tn(gout, x.detach(), with_colsum=want_gb, name="gemm_f32x3_gw")
            gw, gb = res if want_gb else (res, None)
        elif ctx.needs_input_grad[1]:
            gw = _full_precision_matmul(gout.t(), x)
        if want_gb and gb is None:
            gb = gout.sum(0)
        return gx, gw, gb


def _full_precision_matmul(a, b):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        return a @ b
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def linear_f32x3(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _LinearF32x3.apply(x, weight, bias)
