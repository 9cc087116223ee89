"""float32-accurate dense layer on the tensor cores (three TF32 passes).

``linear_f32x3(x, weight, bias)`` computes ``x @ weight.T + bias`` like ``torch.nn.functional.linear``
for float32 CUDA tensors with 32 or 64 input features.  It is meant for the layer that produces
the per-edge weights of a channelwise tensor product from a few edge scalars (the pattern of the
reference's convolution layer, cuequivariance_torch/layers/tp_conv_fully_connected.py:145-152,219-238):
at 1M edges x 2,944 weights that layer is 0.39 TFLOP, an order of magnitude more time than the
tensor product itself when it runs on the CUDA cores.

The forward runs on this library's tcgen05 kernel (``csrc/gemm_f32x3.cu``).  The backward (input
gradient and weight gradient, both reductions over the wide axis) uses device-side torch matmuls:
INTERIM, a fused kernel for them is not written.
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


class _LinearF32x3(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        import ctypes as C

        from . import _lib, profiling

        if not (x.is_cuda and x.dtype == torch.float32 and weight.dtype == torch.float32):
            raise RuntimeError("linear_f32x3 needs float32 CUDA tensors (there is no CPU fallback)")
        if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1] or x.shape[1] not in (32, 64):
            raise ValueError(f"linear_f32x3: x [M, K] and weight [N, K] with K = 32 or 64; got {tuple(x.shape)}, {tuple(weight.shape)}")
        if weight.shape[0] % 4:
            raise ValueError("linear_f32x3: the number of output features must be a multiple of 4")
        xc = x.contiguous()
        hi, lo = split_tf32(weight.detach())
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        status = torch.zeros(1, dtype=torch.int32, device=x.device)
        a = _lib.GemmF32x3Args()
        a.A, a.B_hi, a.B_lo, a.C = xc.data_ptr(), hi.data_ptr(), lo.data_ptr(), out.data_ptr()
        bc = None
        if bias is not None:
            bc = bias.detach().contiguous()
            a.bias = bc.data_ptr()
        a.M, a.N, a.K = xc.shape[0], weight.shape[0], xc.shape[1]
        a.lda, a.ldb, a.ldc = xc.shape[1], hi.shape[1], out.shape[1]
        a.status = status.data_ptr()
        with torch.cuda.device(x.device):
            with profiling.kernel("gemm_f32x3"):
                _lib.check(_lib.lib().cueq_b200_gemm_f32x3(C.byref(a), C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)))
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        ctx.status = status
        return out

    @staticmethod
    def backward(ctx, gout):
        x, weight = ctx.saved_tensors
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            gx = gout @ weight if ctx.needs_input_grad[0] else None
            gw = gout.t() @ x if ctx.needs_input_grad[1] else None
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        gb = gout.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return gx, gw, gb


def linear_f32x3(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return _LinearF32x3.apply(x, weight, bias)
