"""Execution of dense multi-mode tensor products (method ``"fused_tp"``).

Counterpart of the reference's ``SegmentedPolynomialFusedTP``
(cuequivariance_torch/primitives/segmented_polynomial_fused_tp.py:74-262), which hands 3-
and 4-operand products with up to three modes to a closed kernel.

Two routes:

* small products: every mode but the innermost one of the output is flattened into
  segments, which turns the product into a uniform-1d polynomial for the generic CUDA kernel
  (`FusedTPProgram`);
* the fully connected pattern ``uvw,iu,jv,kw+ijk`` with shared weights at sizes where that
  flattening explodes (u*v*nnz paths), `DenseUVW`:
  - bf16/fp16 inputs (or ``options={"tensor_cores": True}``): the tensor-core route.  Per path
    the coupled operand ``Z[(z,k),(u,v)] = sum_ij C[ijk] x1[z,i,u] x2[z,j,v]`` is written in
    bf16 by a CUDA-core kernel and contracted with the weight block by this library's
    TMA + tcgen05 GEMM (float32 accumulation in TMEM); the backward runs two more GEMMs per
    path (weight gradient with both operands MN-major, so nothing is transposed in memory;
    gradient of Z) and a kernel that folds the gradient of Z back onto x1 and x2.  First
    derivatives only.  ``Z`` makes a round trip through HBM; building its tiles directly in
    shared memory inside the GEMM is the remaining step.
  - float32/float64 inputs: INTERIM composite of device-side torch ops with a library GEMM in
    full precision (TF32 off), differentiable to any order; kept because bf16 operands cannot
    meet the float32 tolerance (a split-precision tensor-core variant is not written yet).
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from .executor import Uniform1dProgram
from .polynomial import Polynomial

FLATTEN_LIMIT = 20000  # flattened paths above which the composite route is taken
FUSED_GW = True
FUSED = True  # fully connected tensor-core route: build the coupled operand on chip when the shape allows


def _flatten_all_but_inner(poly: Polynomial) -> Polynomial:
    def fn(d):
        out_sub = d.operand_subscripts[-1] if d.operand_subscripts else ""
        keep = out_sub[-1:] if out_sub else ""
        modes = "".join(m for m in d.modes() if m != keep)
        return d.flatten_modes(modes)

    return poly.map_tensor_products(fn)


def flattened_path_count(poly: Polynomial) -> int:
    n = 0
    for _, d in poly.operations:
        keep = d.operand_subscripts[-1][-1:] if d.operand_subscripts and d.operand_subscripts[-1] else ""
        for p in d.paths:
            dims = d.path_dims(p)
            extra = int(np.prod([v for k, v in dims.items() if k != keep and k not in d.coefficient_subscripts] or [1]))
            n += extra * int(np.count_nonzero(p.coefficients)) if d.coefficient_subscripts else extra
    return n


def _flatten_everything(poly: Polynomial) -> Polynomial:
    def fn(d):
        return d.flatten_modes("".join(d.modes()))

    return poly.map_tensor_products(fn)


def _total_path_count(poly: Polynomial) -> int:
    n = 0
    for _, d in poly.operations:
        for p in d.paths:
            dims = d.path_dims(p)
            extra = int(np.prod([v for k, v in dims.items() if k not in d.coefficient_subscripts] or [1]))
            n += extra * int(np.count_nonzero(p.coefficients)) if d.coefficient_subscripts else extra
    return n


class FusedTPProgram(Uniform1dProgram):
    """Keeps the innermost mode of the output as the channel axis of the generic kernel and
    flattens the rest.  When the segments that remain are not uniform (e.g. a linear map between
    irreps of different multiplicities) every mode is flattened instead, as long as that stays
    below ``FLATTEN_LIMIT`` paths."""

    def __init__(self, polynomial: Polynomial, math_dtype, output_dtype_map=None, name="segmented_polynomial"):
        try:
            super().__init__(_flatten_all_but_inner(polynomial), math_dtype, output_dtype_map, name)
        except ValueError:
            if _total_path_count(polynomial) > FLATTEN_LIMIT:
                raise ValueError(
                    f"{name}: the operands' segments are not uniform and flattening every mode would need "
                    f"{_total_path_count(polynomial)} paths (limit {FLATTEN_LIMIT}); a dense route for this shape is not written"
                )
            super().__init__(_flatten_everything(polynomial), math_dtype, output_dtype_map, name)


def is_fully_connected(poly: Polynomial) -> bool:
    if len(poly.operations) != 1 or poly.num_inputs != 3 or poly.num_outputs != 1:
        return False
    ope, d = poly.operations[0]
    return d.subscripts == "uvw,iu,jv,kw+ijk" and tuple(ope.buffers) == (0, 1, 2, 3)


class _TensorCoreUVW(torch.autograd.Function):
    """``out = sum_paths Z_p W_p`` on the tcgen05 GEMM; see the module docstring."""

    @staticmethod
    def _launch_build(owner, k, x1, x2, Z, B):
        import ctypes as C

        from . import _lib, profiling

        a = owner._fctp_args(k, x1, x2, B)
        a.z = Z.data_ptr()
        a.z_dtype = _lib.BF16
        with profiling.kernel("fctp_build_z"):
            _lib.check(_lib.lib().cueq_b200_fctp_build_z(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    @staticmethod
    def _gemm(A, Bm, Cptr, M, N, K, lda, ldb, ldc, status, accumulate=0, out_bf16=0, a_mn=0, b_mn=0, rows_per_group=1, group_stride=0,
              c_is_zero=0):
        import ctypes as C

        from . import _lib, profiling

        g = _lib.GemmArgs()
        g.A, g.B, g.C = A.data_ptr(), Bm.data_ptr(), Cptr
        g.M, g.N, g.K, g.lda, g.ldb, g.ldc = M, N, K, lda, ldb, ldc
        g.rows_per_group, g.group_stride = rows_per_group, group_stride
        g.accumulate, g.out_bf16, g.a_mn_major, g.b_mn_major = accumulate, out_bf16, a_mn, b_mn
        g.c_is_zero = c_is_zero
        g.status = status.data_ptr()
        with profiling.kernel("gemm_bf16_tcgen05"):
            _lib.check(_lib.lib().cueq_b200_gemm_bf16(C.byref(g), C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    @staticmethod
    def forward(ctx, owner, w, x1, x2):
        d, off = owner.d, owner.offsets
        B = x1.shape[0]
        dev = x1.device
        from . import _lib

        status = _lib.status_word(dev)
        if FUSED and owner._fused_tasks() is not None:
            out = owner._fused_forward(w, x1, x2, status)
            ctx.owner, ctx.status = owner, status
            ctx.save_for_backward(w, x1, x2)
            return out.to(x1.dtype)
        x1c, x2c = owner._as_kernel_input(x1), owner._as_kernel_input(x2)
        out = torch.zeros((B, owner.out_size), dtype=torch.float32, device=dev)
        seen = set()
        for k, p in enumerate(d.paths):
            sw, s1, s2, so = p.indices
            U, V, Wd = d.operands[0].segments[sw]
            d3 = p.coefficients.shape[2]
            rows = B * d3
            Z = torch.empty((rows, U * V), dtype=torch.bfloat16, device=dev)
            _TensorCoreUVW._launch_build(owner, k, x1c, x2c, Z, B)
            WT = w[0, off[0][sw] : off[0][sw] + U * V * Wd].reshape(U * V, Wd).t().contiguous().to(torch.bfloat16)
            cptr = out.data_ptr() + 4 * off[3][so]
            _TensorCoreUVW._gemm(Z, WT, cptr, rows, Wd, U * V, U * V, U * V, Wd, status, accumulate=1 if so in seen else 0,
                                 rows_per_group=d3, group_stride=owner.out_size)
            seen.add(so)
        ctx.owner, ctx.status = owner, status
        ctx.save_for_backward(w, x1, x2)
        return out.to(x1.dtype)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gout):
        import ctypes as C

        from . import _lib, profiling

        owner = ctx.owner
        w, x1, x2 = ctx.saved_tensors
        d, off = owner.d, owner.offsets
        B, dev = x1.shape[0], x1.device
        need_w, need_x1, need_x2 = ctx.needs_input_grad[1], ctx.needs_input_grad[2], ctx.needs_input_grad[3]
        status = ctx.status
        fused_x = FUSED and owner._fused_tasks() is not None and owner._fused_units(1) is not None and owner._fused_wunits() is not None
        gx1f = gx2f = gwf = None
        if fused_x and (need_x1 or need_x2 or need_w):
            gout16 = gout.to(torch.bfloat16).contiguous()
            x1b, x2b = x1.to(torch.bfloat16).contiguous(), x2.to(torch.bfloat16).contiguous()
            if need_w and FUSED_GW:
                gwf = owner._fused_gw(w, x1b, x2b, gout16, status)
                need_w = False
            if need_x1:
                gx1f = owner._fused_gx(1, w.reshape(-1, 64).to(torch.bfloat16).contiguous(), x2b, gout16, status)
            if need_x2:
                wt = w.reshape(-1, 64, 64, 64).transpose(1, 2).reshape(-1, 64).to(torch.bfloat16).contiguous()
                gx2f = owner._fused_gx(2, wt, x1b, gout16, status)
            need_x1 = need_x2 = False
        x1c, x2c = owner._as_kernel_input(x1), owner._as_kernel_input(x2)
        gw = torch.zeros((1, w.shape[1]), dtype=torch.float32, device=dev) if need_w else None
        gx1 = torch.zeros(x1.shape, dtype=torch.float32, device=dev) if need_x1 else None
        gx2 = torch.zeros(x2.shape, dtype=torch.float32, device=dev) if need_x2 else None
        for k, p in enumerate(d.paths):
            sw, s1, s2, so = p.indices
            U, V, Wd = d.operands[0].segments[sw]
            if not (need_w or need_x1 or need_x2):
                break
            d3 = p.coefficients.shape[2]
            rows = B * d3
            rows_pad = (rows + 63) // 64 * 64
            G = torch.zeros((rows_pad, Wd), dtype=torch.bfloat16, device=dev)
            G[:rows] = gout[:, off[3][so] : off[3][so] + d3 * Wd].reshape(rows, Wd)
            if need_w:
                Z = torch.empty((rows_pad, U * V), dtype=torch.bfloat16, device=dev)
                if rows_pad > rows:
                    Z[rows:].zero_()
                _TensorCoreUVW._launch_build(owner, k, x1c, x2c, Z, B)
                gwp = gw[0, off[0][sw] : off[0][sw] + U * V * Wd]
                # gW[(uv), w] = sum_(z,k) Z[(z,k),(uv)] G[(z,k),w]: both operands are stored [K][M or N]
                _TensorCoreUVW._gemm(Z, G, gwp.data_ptr(), U * V, Wd, rows_pad, U * V, Wd, Wd, status, a_mn=1, b_mn=1, c_is_zero=1)
                del Z
            if need_x1 or need_x2:
                W16 = w[0, off[0][sw] : off[0][sw] + U * V * Wd].reshape(U * V, Wd).contiguous().to(torch.bfloat16)
                gZ = torch.empty((rows, U * V), dtype=torch.bfloat16, device=dev)
                _TensorCoreUVW._gemm(G, W16, gZ.data_ptr(), rows, U * V, Wd, Wd, Wd, U * V, status, out_bf16=1)
                a = owner._fctp_args(k, x1c, x2c, B)
                a.z, a.z_dtype = gZ.data_ptr(), _lib.BF16
                a.gx1 = gx1.data_ptr() if need_x1 else None
                a.gx2 = gx2.data_ptr() if need_x2 else None
                with profiling.kernel("fctp_consume_gz"):
                    _lib.check(_lib.lib().cueq_b200_fctp_consume_gz(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
                del gZ
        if gwf is not None:
            gw, need_w = gwf, True
        if gx1f is not None:
            gx1, need_x1 = gx1f, True
        if gx2f is not None:
            gx2, need_x2 = gx2f, True
        return (None, gw.to(w.dtype) if need_w else None, gx1.to(x1.dtype) if need_x1 else None,
                gx2.to(x2.dtype) if need_x2 else None)


class DenseUVW:
    """Dense route for ``uvw,iu,jv,kw+ijk`` (see the module docstring)."""

    def __init__(self, polynomial: Polynomial, math_dtype: Optional[torch.dtype], options: Optional[dict] = None):
        _, d = polynomial.operations[0]
        self.d = d
        self.math_dtype = math_dtype
        self.force_tc = bool((options or {}).get("tensor_cores", False))
        self._cg = {}
        self.offsets = [op.offsets() for op in d.operands]
        self.out_size = d.operands[3].size
        self._coef = {}

    def _c(self, k, device, dtype):
        key = (k, device, dtype)
        t = self._coef.get(key)
        if t is None:
            t = torch.tensor(self.d.paths[k].coefficients, dtype=dtype, device=device)
            self._coef[key] = t
        return t

    # -- tensor-core route ---------------------------------------------------------------------
    def _tc_applicable(self, w, x1, x2) -> bool:
        if w.shape[0] != 1 or x1.shape[0] != x2.shape[0] or x1.shape[0] == 0:
            return False
        if not (self.force_tc or x1.dtype in (torch.bfloat16, torch.float16)):
            return False
        for p in self.d.paths:
            U, V, Wd = self.d.operands[0].segments[p.indices[0]]
            if (U * V) % 128 or Wd % 64 or V % 2 or max(p.coefficients.shape) > 7:
                return False
        return True

    # -- fused route: coupled operand built in shared memory ------------------------------------
    def _fused_tasks(self):
        """Task table for the fused kernels, or None if the shape is outside what they cover
        (all multiplicities 64, irrep dimensions 1/3/5, at most 4 paths per output irrep)."""
        if hasattr(self, "_tasks"):
            return self._tasks
        from . import _lib

        d, off = self.d, self.offsets
        self._tasks = None
        by_out = {}
        for p in d.paths:
            sw, s1, s2, so = p.indices
            if tuple(d.operands[0].segments[sw]) != (64, 64, 64):
                return None
            d1, d2, d3 = p.coefficients.shape
            if d1 not in (1, 3, 5) or d2 not in (1, 3, 5) or off[0][sw] % 64:
                return None
            by_out.setdefault(so, []).append(p)
        tasks = []
        for so, paths in sorted(by_out.items()):
            if len(paths) > 4:
                return None
            d3 = paths[0].coefficients.shape[2]
            for k in range(d3):
                t = _lib.FctpFusedTask()
                t.out_off, t.num_paths = off[3][so] + k * 64, len(paths)
                for q, p in enumerate(paths):
                    sw, s1, s2, _ = p.indices
                    fp = t.paths[q]
                    fp.off1, fp.off2 = off[1][s1], off[2][s2]
                    fp.d1, fp.d2, fp.w_row0 = p.coefficients.shape[0], p.coefficients.shape[1], off[0][sw] // 64
                    for i in range(fp.d1):
                        for j in range(fp.d2):
                            fp.c[i * 5 + j] = float(p.coefficients[i, j, k])
                tasks.append(t)
        if len(tasks) > 12 or len(by_out) != d.operands[3].num_segments:
            return None
        self._tasks = (_lib.FctpFusedTask * len(tasks))(*tasks)
        return self._tasks

    def _fused_units(self, which: int):
        """Unit table of the fused gradient kernel for x1 (``which`` = 1) or x2 (2)."""
        key = f"_units{which}"
        if hasattr(self, key):
            return getattr(self, key)
        from . import _lib

        d, off = self.d, self.offsets
        units = []
        for p in d.paths:
            sw, s1, s2, so = p.indices
            d1, d2, d3 = p.coefficients.shape
            for k0 in range(0, d3, 2):
                u = _lib.FctpFusedUnit()
                u.w_row0 = off[0][sw] // 64
                u.nk = min(2, d3 - k0)
                if which == 1:
                    u.offa, u.offb, u.da, u.db = off[1][s1], off[2][s2], d1, d2
                else:
                    u.offa, u.offb, u.da, u.db = off[2][s2], off[1][s1], d2, d1
                for kq in range(u.nk):
                    u.goff[kq] = off[3][so] + (k0 + kq) * 64
                    for i in range(d1):
                        for j in range(d2):
                            c = float(p.coefficients[i, j, k0 + kq])
                            if which == 1:
                                u.c[kq][i * 5 + j] = c
                            else:
                                u.c[kq][j * 5 + i] = c
                units.append(u)
        arr = (_lib.FctpFusedUnit * len(units))(*units) if len(units) <= 32 else None
        setattr(self, key, arr)
        return arr

    def _fused_gx(self, which, w16, xb, gout16, status):
        import ctypes as C

        from . import _lib, profiling

        units = self._fused_units(which)
        B = xb.shape[0]
        gxa = torch.zeros((B, xb.shape[1]), dtype=torch.float32, device=xb.device)
        a = _lib.FctpFusedGxArgs()
        a.xb, a.gout, a.w, a.gxa = xb.data_ptr(), gout16.data_ptr(), w16.data_ptr(), gxa.data_ptr()
        a.ldb, a.ldg, a.lda, a.batch, a.w_rows = xb.shape[1], gout16.shape[1], gxa.shape[1], B, w16.shape[0]
        a.num_units = len(units)
        a.units = C.cast(units, C.POINTER(_lib.FctpFusedUnit))
        a.status = status.data_ptr()
        with profiling.kernel(f"fctp_fused_gx{which}"):
            _lib.check(_lib.lib().cueq_b200_fctp_fused_gx(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return gxa

    def _fused_wunits(self):
        if hasattr(self, "_wunits"):
            return self._wunits
        from . import _lib

        d, off = self.d, self.offsets
        units = []
        for p in d.paths:
            sw, s1, s2, so = p.indices
            d1, d2, d3 = p.coefficients.shape
            for k in range(d3):
                u = _lib.FctpFusedWUnit()
                u.off1, u.off2, u.d1, u.d2 = off[1][s1], off[2][s2], d1, d2
                u.w_row0, u.goff = off[0][sw] // 64, off[3][so] + k * 64
                for i in range(d1):
                    for j in range(d2):
                        u.c[i * 5 + j] = float(p.coefficients[i, j, k])
                units.append(u)
        self._wunits = (_lib.FctpFusedWUnit * len(units))(*units) if len(units) <= 48 else None
        return self._wunits

    def _fused_gw(self, w, x1b, x2b, gout16, status):
        import ctypes as C

        from . import _lib, profiling

        units = self._fused_wunits()
        gw = torch.zeros((w.numel() // 64, 64), dtype=torch.float32, device=w.device)
        a = _lib.FctpFusedGwArgs()
        a.x1, a.x2, a.gout, a.gw = x1b.data_ptr(), x2b.data_ptr(), gout16.data_ptr(), gw.data_ptr()
        a.ld1, a.ld2, a.ldg, a.batch, a.w_rows = x1b.shape[1], x2b.shape[1], gout16.shape[1], x1b.shape[0], gw.shape[0]
        a.num_units = len(units)
        a.units = C.cast(units, C.POINTER(_lib.FctpFusedWUnit))
        a.status = status.data_ptr()
        with profiling.kernel("fctp_fused_gw"):
            _lib.check(_lib.lib().cueq_b200_fctp_fused_gw(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return gw.reshape(1, -1)

    def _fused_forward(self, w, x1, x2, status):
        import ctypes as C

        from . import _lib, profiling

        tasks = self._fused_tasks()
        B = x1.shape[0]
        x1c, x2c = x1.to(torch.bfloat16).contiguous(), x2.to(torch.bfloat16).contiguous()
        w16 = w.reshape(-1, 64).to(torch.bfloat16).contiguous()
        out = torch.empty((B, self.out_size), dtype=torch.float32, device=x1.device)
        a = _lib.FctpFusedArgs()
        a.x1, a.x2, a.w, a.out = x1c.data_ptr(), x2c.data_ptr(), w16.data_ptr(), out.data_ptr()
        a.ld1, a.ld2, a.ldo, a.batch, a.w_rows = x1c.shape[1], x2c.shape[1], out.shape[1], B, w16.shape[0]
        a.out_dtype, a.num_tasks = _lib.F32, len(tasks)
        a.tasks = C.cast(tasks, C.POINTER(_lib.FctpFusedTask))
        a.status = status.data_ptr()
        with profiling.kernel("fctp_fused_forward"):
            _lib.check(_lib.lib().cueq_b200_fctp_fused_forward(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out

    @staticmethod
    def _as_kernel_input(x):
        if x.dtype in (torch.float32, torch.bfloat16):
            return x.contiguous()
        return x.float().contiguous()

    def _fctp_args(self, k, x1, x2, B):
        import ctypes as C

        from . import _lib
        from .executor import dtype_code

        d, off, p = self.d, self.offsets, self.d.paths[k]
        sw, s1, s2, so = p.indices
        U, V, _ = d.operands[0].segments[sw]
        d1, d2, d3 = p.coefficients.shape
        cg = self._cg.get(k)
        if cg is None:
            flat = [float(v) for v in p.coefficients.reshape(-1)]
            cg = (C.c_float * len(flat))(*flat)
            self._cg[k] = cg
        a = _lib.FctpArgs()
        a.x1, a.x2 = x1.data_ptr(), x2.data_ptr()
        a.cg = C.cast(cg, C.POINTER(C.c_float))
        a.ld1, a.ld2, a.batch = x1.shape[1], x2.shape[1], B
        a.off1, a.off2 = off[1][s1], off[2][s2]
        a.d1, a.d2, a.d3, a.U, a.V = d1, d2, d3, U, V
        a.x_dtype = dtype_code(x1.dtype)
        return a

    def __call__(self, inputs: List[torch.Tensor]) -> List[torch.Tensor]:
        w, x1, x2 = inputs
        if w.device.type != "cuda":
            raise RuntimeError("cuequivariance_b200 executes on CUDA devices only (there is no CPU fallback)")
        if self._tc_applicable(w, x1, x2):
            if x1.dtype != x2.dtype:
                x2 = x2.to(x1.dtype)
            return [_TensorCoreUVW.apply(self, w, x1, x2)]
        io = x1.dtype
        md = self.math_dtype or (io if io in (torch.float32, torch.float64) else torch.float32)
        d, off = self.d, self.offsets
        B = max(x1.shape[0], x2.shape[0], w.shape[0])
        pieces = [None] * d.operands[3].num_segments
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            for k, p in enumerate(d.paths):
                sw, s1, s2, so = p.indices
                u, v, wd = d.operands[0].segments[sw]
                d1, d2, d3 = p.coefficients.shape
                a = x1[:, off[1][s1] : off[1][s1] + d1 * u].reshape(-1, d1, u).to(md)
                b = x2[:, off[2][s2] : off[2][s2] + d2 * v].reshape(-1, d2, v).to(md)
                z = torch.einsum("ijk,ziu,zjv->zkuv", self._c(k, x1.device, md), a, b)
                wk = w[:, off[0][sw] : off[0][sw] + u * v * wd].to(md)
                if wk.shape[0] == 1:
                    r = (z.reshape(-1, u * v) @ wk.reshape(u * v, wd)).reshape(-1, d3 * wd)
                else:
                    r = torch.einsum("zkq,zqw->zkw", z.reshape(z.shape[0], d3, u * v), wk.reshape(-1, u * v, wd)).reshape(-1, d3 * wd)
                pieces[so] = r if pieces[so] is None else pieces[so] + r
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        cols = []
        for s, seg in enumerate(d.operands[3].segments):
            cols.append(pieces[s] if pieces[s] is not None else x1.new_zeros(B, int(np.prod(seg)), dtype=md))
        return [torch.cat(cols, dim=1).to(io)]
