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
  - float32 inputs: the same decomposition in float32 accuracy.  ``Z`` is written in float32 (the
    paths that feed one output irrep side by side, so one GEMM per output component contracts them
    all) and contracted by this library's three-pass TF32 tcgen05 GEMMs (``dense.gemm_f32x3`` and
    its row-reduction twin for the weight gradient); differentiable to any order, because every
    derivative of a tri-linear map is again one of the same four contractions.
  - float64 inputs and per-sample weights: the generic kernel on the fully flattened product.
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
                gx1f = owner._fused_gx(1, owner._weights_bf16(w, False), x2b, gout16, status)
            if need_x2:
                gx2f = owner._fused_gx(2, owner._weights_bf16(w, True), x1b, gout16, status)
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
        self._flat = {}
        self._wcache = {}

    def _weights_bf16(self, w: torch.Tensor, transposed: bool) -> torch.Tensor:
        """The shared weights as bf16 rows of 64, in ``[u][v][w]`` order or (``transposed``) ``[v][u][w]``.  The same
        weight tensor is used by every call of a step and changes only when the optimizer updates it, so the
        converted copies are kept until the tensor's version counter moves (or another tensor is passed)."""
        key = (w.data_ptr(), w._version, tuple(w.shape), w.dtype, transposed)
        hit = self._wcache.get(transposed)
        if hit is not None and hit[0] == key:
            return hit[1]
        if transposed:
            t = w.detach().reshape(-1, 64, 64, 64).transpose(1, 2).reshape(-1, 64).to(torch.bfloat16).contiguous()
        else:
            t = w.detach().reshape(-1, 64).to(torch.bfloat16).contiguous()
        self._wcache[transposed] = (key, t)
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
        w16 = self._weights_bf16(w, False)
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
        if x1.dtype == torch.float32 and x2.dtype == torch.float32 and w.dtype == torch.float32 and w.shape[0] == 1 \
                and self.math_dtype in (None, torch.float32) and self._f32_applicable():
            B = max(x1.shape[0], x2.shape[0])
            x1 = x1.expand(B, -1) if x1.shape[0] != B else x1
            x2 = x2.expand(B, -1) if x2.shape[0] != B else x2
            return [_DenseOut.apply(self, w, x1.contiguous(), x2.contiguous())]
        return self._flattened(x1.dtype)(inputs)

    # -- float32 route: float32-accurate tensor-core GEMMs on the coupled operand -----------------
    def _f32_applicable(self) -> bool:
        return all(self.d.operands[0].segments[p.indices[0]][1] % 2 == 0 and max(p.coefficients.shape) <= 7 for p in self.d.paths)

    def _flattened(self, io_dtype):
        """float64 operands, per-sample weights and shapes the dense kernels do not take run on the
        generic kernel with every mode but the output's innermost one flattened into paths: correct
        for any shape, slow for large multiplicities (hundreds of thousands of paths)."""
        md = self.math_dtype or (io_dtype if io_dtype in (torch.float32, torch.float64) else torch.float32)
        prog = self._flat.get(md)
        if prog is None:
            import warnings

            from .executor import evaluate
            from .polynomial import Operation

            poly = Polynomial(list(self.d.operands[:3]), [self.d.operands[3]], [(Operation((0, 1, 2, 3)), self.d)])
            n = flattened_path_count(poly)
            if n > FLATTEN_LIMIT:
                warnings.warn(f"fully connected product: this call (dtype {io_dtype}, math {md}) is outside the dense kernels and runs "
                              f"on the generic kernel with {n} flattened paths")
            fp = FusedTPProgram(poly, md, None, "fully_connected_flattened")
            prog = lambda xs, fp=fp: evaluate(fp, list(xs), {}, {}, {}, None)  # noqa: E731
            self._flat[md] = prog
        return prog

    def _by_output(self):
        if not hasattr(self, "_by_out"):
            by = {}
            for k, p in enumerate(self.d.paths):
                by.setdefault(p.indices[3], []).append(k)
            self._by_out = by
        return self._by_out

    @staticmethod
    def _pad32(n: int) -> int:
        return (n + 31) // 32 * 32

    def _build_f32(self, k, x1, x2, Z, ldz, col0):
        """Z[:, col0 : col0 + U*V] (rows (z, k), pitch ldz) = coupled operand of path k, float32."""
        import ctypes as C

        from . import _lib, profiling

        a = self._fctp_args(k, x1, x2, x1.shape[0])
        a.z = Z.data_ptr() + 4 * col0
        a.z_dtype, a.ldz = _lib.F32, ldz
        with profiling.kernel("fctp_build_z"):
            _lib.check(_lib.lib().cueq_b200_fctp_build_z(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def _chunk(self, B: int, row_floats: int) -> int:
        """Samples per pass so that the coupled operand of a pass stays below about 4 GB."""
        return max(128, min(B, int(1e9 // max(1, row_floats)) // 128 * 128))

    def map_out(self, w, x1, x2):
        """out = F(w, x1, x2): per output irrep one coupled operand [(z, k), sum of the paths' (u, v)] and one
        GEMM per component k against the stacked weight blocks."""
        from .dense import gemm_f32x3, split_tf32

        d, off = self.d, self.offsets
        B, dev = x1.shape[0], x1.device
        out = torch.zeros((B, self.out_size), dtype=torch.float32, device=dev)
        for so, ks in sorted(self._by_output().items()):
            d3, Wd = d.operands[3].segments[so][0], d.operands[3].segments[so][1]
            cols = [self._pad32(d.operands[0].segments[d.paths[k].indices[0]][0] * d.operands[0].segments[d.paths[k].indices[0]][1]) for k in ks]
            K = sum(cols)
            Wp = -(-Wd // 4) * 4
            WT = torch.zeros((Wp, K), dtype=torch.float32, device=dev)      # stacked W_p^T, zero rows/columns as padding
            c0 = 0
            for k, ck in zip(ks, cols):
                sw = d.paths[k].indices[0]
                U, V, _ = d.operands[0].segments[sw]
                WT[:Wd, c0 : c0 + U * V] = w[0, off[0][sw] : off[0][sw] + U * V * Wd].reshape(U * V, Wd).t()
                c0 += ck
            WT_split = split_tf32(WT)                                        # one split for every component and chunk
            step = self._chunk(B, d3 * K)
            for b0 in range(0, B, step):
                b1 = min(B, b0 + step)
                padded = any(c != d.operands[0].segments[d.paths[k].indices[0]][0] * d.operands[0].segments[d.paths[k].indices[0]][1] for k, c in zip(ks, cols))
                Z = (torch.zeros if padded else torch.empty)(((b1 - b0) * d3, K), dtype=torch.float32, device=dev)
                c0 = 0
                for k, ck in zip(ks, cols):
                    self._build_f32(k, x1[b0:b1], x2[b0:b1], Z, K, c0)
                    c0 += ck
                Z3 = Z.view(b1 - b0, d3, K)
                for kk in range(d3):
                    o = off[3][so] + kk * Wd
                    if Wp == Wd:
                        gemm_f32x3(Z3[:, kk, :], WT, name="fctp_f32_forward", out=out[b0:b1, o : o + Wd], b_split=WT_split)
                    else:
                        out[b0:b1, o : o + Wd] = gemm_f32x3(Z3[:, kk, :], WT, name="fctp_f32_forward", b_split=WT_split)[:, :Wd]
                del Z, Z3
        return out

    def map_w(self, x1, x2, g):
        """dPhi/dw: per path  gW[(u,v), w] = sum_(z,k) Z[(z,k),(u,v)] g[z, k, w]  (reduction over rows)."""
        from .dense import gemm_f32x3_tn

        d, off = self.d, self.offsets
        B, dev = x1.shape[0], x1.device
        gw = torch.zeros((1, d.operands[0].size), dtype=torch.float32, device=dev)
        for k, p in enumerate(d.paths):
            sw, _, _, so = p.indices
            U, V, Wd = d.operands[0].segments[sw]
            d3 = p.coefficients.shape[2]
            K = self._pad32(U * V)
            Wp = -(-Wd // 4) * 4
            acc = torch.zeros((K, Wp), dtype=torch.float32, device=dev)
            step = self._chunk(B, d3 * K)
            for b0 in range(0, B, step):
                b1 = min(B, b0 + step)
                Z = (torch.zeros if K != U * V else torch.empty)(((b1 - b0) * d3, K), dtype=torch.float32, device=dev)
                self._build_f32(k, x1[b0:b1], x2[b0:b1], Z, K, 0)
                Z3 = Z.view(b1 - b0, d3, K)
                for kk in range(d3):
                    o = off[3][so] + kk * Wd
                    gk = g[b0:b1, o : o + Wd]
                    if Wp != Wd:
                        gk = torch.nn.functional.pad(gk, (0, Wp - Wd))
                    gemm_f32x3_tn(Z3[:, kk, :], gk, name="fctp_f32_gw", out=acc)
                del Z, Z3
            gw[0, off[0][sw] : off[0][sw] + U * V * Wd] = acc[: U * V, :Wd].reshape(-1)
        return gw

    def map_x(self, w, x1, x2, g):
        """(dPhi/dx1, dPhi/dx2): per path gZ = g W^T by one GEMM per component, folded against the other operand."""
        import ctypes as C

        from . import _lib, profiling
        from .dense import gemm_f32x3, split_tf32

        d, off = self.d, self.offsets
        B, dev = x1.shape[0], x1.device
        gx1 = torch.zeros(x1.shape, dtype=torch.float32, device=dev)
        gx2 = torch.zeros(x2.shape, dtype=torch.float32, device=dev)
        for k, p in enumerate(d.paths):
            sw, _, _, so = p.indices
            U, V, Wd = d.operands[0].segments[sw]
            d3 = p.coefficients.shape[2]
            N = -(-U * V // 4) * 4
            Kw = self._pad32(Wd)
            Wk = w[0, off[0][sw] : off[0][sw] + U * V * Wd].reshape(U * V, Wd)
            if Kw != Wd or N != U * V:
                Wk = torch.nn.functional.pad(Wk, (0, Kw - Wd, 0, N - U * V))
            Wk = Wk.contiguous()
            Wk_split = split_tf32(Wk)                                        # one split for every component and chunk
            step = self._chunk(B, d3 * N)
            for b0 in range(0, B, step):
                b1 = min(B, b0 + step)
                gZ = torch.empty(((b1 - b0) * d3, N), dtype=torch.float32, device=dev)
                gZ3 = gZ.view(b1 - b0, d3, N)
                for kk in range(d3):
                    o = off[3][so] + kk * Wd
                    gk = g[b0:b1, o : o + Wd]
                    if Kw != Wd:
                        gk = torch.nn.functional.pad(gk, (0, Kw - Wd))
                    gemm_f32x3(gk, Wk, name="fctp_f32_gx", out=gZ3[:, kk, :], b_split=Wk_split)
                a = self._fctp_args(k, x1[b0:b1], x2[b0:b1], b1 - b0)
                a.z, a.z_dtype, a.ldz = gZ.data_ptr(), _lib.F32, N
                a.gx1, a.gx2 = gx1[b0:b1].data_ptr(), gx2[b0:b1].data_ptr()
                with profiling.kernel("fctp_consume_gz"):
                    _lib.check(_lib.lib().cueq_b200_fctp_consume_gz(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
                del gZ, gZ3
        return gx1, gx2


# The fully connected product is linear in each of (w, x1, x2); with Phi(w, x1, x2, g) = <g, F(w, x1, x2)> every
# derivative of every order is one of four contractions of Phi with three of its arguments: F itself and the
# partial derivatives of Phi with respect to w, x1 and x2.  Each is a function below whose backward is made of
# the others, so the float32 dense route is differentiable to any order on this library's kernels alone.
class _DenseOut(torch.autograd.Function):
    @staticmethod
    def forward(ctx, owner, w, x1, x2):
        ctx.owner = owner
        ctx.save_for_backward(w, x1, x2)
        return owner.map_out(w.detach(), x1.detach(), x2.detach())

    @staticmethod
    def backward(ctx, g):
        w, x1, x2 = ctx.saved_tensors
        g = g.contiguous()
        gw = _DenseGw.apply(ctx.owner, x1, x2, g) if ctx.needs_input_grad[1] else None
        gx1 = gx2 = None
        if ctx.needs_input_grad[2] or ctx.needs_input_grad[3]:
            gx1, gx2 = _DenseGx.apply(ctx.owner, w, x1, x2, g)
        return None, gw, gx1 if ctx.needs_input_grad[2] else None, gx2 if ctx.needs_input_grad[3] else None


class _DenseGw(torch.autograd.Function):
    @staticmethod
    def forward(ctx, owner, x1, x2, g):
        ctx.owner = owner
        ctx.save_for_backward(x1, x2, g)
        return owner.map_w(x1.detach(), x2.detach(), g.detach())

    @staticmethod
    def backward(ctx, tw):
        x1, x2, g = ctx.saved_tensors
        tw = tw.contiguous()
        gx1 = gx2 = gg = None
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            gx1, gx2 = _DenseGx.apply(ctx.owner, tw, x1, x2, g)
        if ctx.needs_input_grad[3]:
            gg = _DenseOut.apply(ctx.owner, tw, x1, x2)
        return None, gx1 if ctx.needs_input_grad[1] else None, gx2 if ctx.needs_input_grad[2] else None, gg


class _DenseGx(torch.autograd.Function):
    @staticmethod
    def forward(ctx, owner, w, x1, x2, g):
        ctx.owner = owner
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(w, x1, x2, g)
        return owner.map_x(w.detach(), x1.detach(), x2.detach(), g.detach())

    @staticmethod
    def backward(ctx, t1, t2):
        w, x1, x2, g = ctx.saved_tensors
        owner = ctx.owner
        need_w, need_1, need_2, need_g = ctx.needs_input_grad[1:5]
        gw = g1 = g2 = gg = None

        def add(a, b):
            return b if a is None else (a if b is None else a + b)

        if t1 is not None:          # <t1, dPhi/dx1(w, x2, g)> = Phi(w, t1, x2, g)
            t1 = t1.contiguous()
            if need_w:
                gw = add(gw, _DenseGw.apply(owner, t1, x2, g))
            if need_2:
                g2 = add(g2, _DenseGx.apply(owner, w, t1, x2, g)[1])
            if need_g:
                gg = add(gg, _DenseOut.apply(owner, w, t1, x2))
        if t2 is not None:          # <t2, dPhi/dx2(w, x1, g)> = Phi(w, x1, t2, g)
            t2 = t2.contiguous()
            if need_w:
                gw = add(gw, _DenseGw.apply(owner, x1, t2, g))
            if need_1:
                g1 = add(g1, _DenseGx.apply(owner, w, x1, t2, g)[0])
            if need_g:
                gg = add(gg, _DenseOut.apply(owner, w, x1, t2))
        return None, gw, g1, g2, gg
