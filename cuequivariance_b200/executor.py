"""Host side of the executor: lowering of a polynomial to launch tables, buffer
addressing modes, and the autograd rule that evaluates derivatives as polynomials.

The lowering reproduces what the reference front-end sends to its closed kernel
(cuequivariance_torch/primitives/segmented_polynomial_uniform_1d.py:105-218): flatten the
coefficient modes, squeeze extent-1 modes, require scalar coefficients and a single
uniform mode, then serialise segment counts, operation buffer ids, path indices and
path coefficients.  Buffer addressing follows :242-292 (shared / batched / indexed).

Derivatives: the backward of a polynomial call is another polynomial call (same
executor, cotangents as extra inputs, gather and scatter roles swapped), so gradients of
any order come from one mechanism (the reference's JAX front-end does the same,
cuequivariance_jax/segmented_polynomials/segmented_polynomial.py:552-673).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from .polynomial import Polynomial

_TORCH_TO_CODE = {
    torch.float32: _lib.F32,
    torch.float64: _lib.F64,
    torch.bfloat16: _lib.BF16,
    torch.float16: _lib.F16,
}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _TORCH_TO_CODE[dt]
    except KeyError:
        raise ValueError(f"unsupported tensor dtype {dt}") from None


@dataclass(frozen=True)
class BufferSpec:
    """Addressing of one buffer for one call."""

    mode: int                        # _lib.SHARED / BATCHED / INDEXED
    rows: int
    index: Optional[torch.Tensor]    # [batch] int32/int64 when INDEXED

    def key(self):
        return (self.mode, self.rows, None if self.index is None else (self.index.data_ptr(), self.index.dtype))


@dataclass(frozen=True)
class CallConfig:
    """``layouts[b]`` (b over inputs then outputs) is None when buffer b is exchanged in the
    polynomial's own component-major (ir_mul) layout, or a tuple of ``(mul, dim)`` blocks
    when the caller holds it channel-major (mul_ir): specialised kernels fold the
    transposition into their addressing, the generic path transposes explicitly."""

    batch: int
    inputs: Tuple[BufferSpec, ...]
    outputs: Tuple[BufferSpec, ...]
    layouts: Tuple[Optional[tuple], ...] = ()

    def layout(self, b: int) -> Optional[tuple]:
        return self.layouts[b] if self.layouts else None


class Uniform1dProgram:
    """A polynomial lowered to the uniform-1d form plus its native plan.

    Owns: the flattened polynomial, the native plan handle, one device copy of the plan
    tables per device, and the programs of its derivatives (built on demand).
    """

    def __init__(self, polynomial: Polynomial, math_dtype: torch.dtype, output_dtype_map: Optional[Sequence[int]] = None,
                 name: str = "segmented_polynomial"):
        if math_dtype not in (torch.float32, torch.float64):
            raise ValueError(f"math_dtype must be float32 or float64 for method 'uniform_1d'; got {math_dtype}")
        self.name = name
        self.math_dtype = math_dtype
        self.original = polynomial
        try:
            flat = polynomial.flatten_coefficient_modes()
        except ValueError as e:
            raise ValueError(
                "Failed to prepare polynomial for method 'uniform_1d': coefficient modes could not be flattened.\n"
                f"{e}\n{polynomial}"
            ) from e
        flat = flat.squeeze_modes()
        extent = None
        for o in flat.operands:
            if o.ndim not in (0, 1):
                raise ValueError("For method 'uniform_1d', only 0D (scalar) or 1D operands are supported.")
            if o.num_segments and o.uniform_shape() is None:
                raise ValueError("For method 'uniform_1d', all segments of a given operand must have the same shape.")
            if o.ndim == 1 and o.num_segments:
                (x,) = o.uniform_shape()
                if extent is None:
                    extent = x
                elif extent != x:
                    raise ValueError("For method 'uniform_1d', all 1D operands must share the same segment extent.")
        for _, stp in flat.operations:
            if stp.coefficient_subscripts != "":
                raise ValueError("In method 'uniform_1d', coefficients must be scalar.")
        self.flat = flat
        self.extent = extent or 1
        self.num_inputs, self.num_outputs = flat.num_inputs, flat.num_outputs
        default_map = [0 if self.num_inputs >= 1 else -1] * self.num_outputs
        self.output_dtype_map = list(default_map if output_dtype_map is None else output_dtype_map)
        self.buffer_dim = [o.ndim for o in flat.operands]
        self.buffer_num_segments = [o.num_segments for o in flat.operands]
        self.row_sizes = [o.size for o in flat.operands]
        self._plan = None
        self._tables_host: Optional[torch.Tensor] = None
        self._tables_dev: Dict[torch.device, torch.Tensor] = {}
        self._derivatives: Dict[tuple, "Uniform1dProgram"] = {}
        self._special = None  # filled by specialised-kernel matchers

    # -- native plan -------------------------------------------------------------------
    def serialised(self) -> dict:
        """The lists the reference front-end would hand to its op (names as in
        segmented_polynomial_uniform_1d.py:188-218)."""
        ops = self.flat.operations
        return dict(
            operand_extent=self.extent,
            num_inputs=self.num_inputs,
            num_outputs=self.num_outputs,
            buffer_dim=list(self.buffer_dim),
            buffer_num_segments=list(self.buffer_num_segments),
            num_operations=len(ops),
            num_operands=[len(o.buffers) for o, _ in ops],
            operations=[b for o, _ in ops for b in o.buffers],
            num_paths=[d.num_paths for _, d in ops],
            path_indices=[i for _, d in ops for p in d.paths for i in p.indices],
            path_coefficients=[float(p.coefficients) for _, d in ops for p in d.paths],
        )

    def plan(self):
        if self._plan is None:
            s = self.serialised()
            self._keep = [
                _lib.int32_array(s["buffer_dim"]), _lib.int32_array(s["buffer_num_segments"]),
                _lib.int32_array(s["num_operands"]), _lib.int32_array(s["operations"]),
                _lib.int32_array(s["num_paths"]), _lib.int32_array(s["path_indices"]),
                _lib.double_array(s["path_coefficients"]),
            ]
            k = self._keep
            desc = _lib.U1dDesc(
                s["operand_extent"], s["num_inputs"], s["num_outputs"], k[0], k[1], s["num_operations"],
                k[2], k[3], k[4], k[5], k[6], dtype_code(self.math_dtype),
            )
            handle = C.c_void_p()
            _lib.check(_lib.lib().cueq_b200_u1d_plan_create(C.byref(desc), C.byref(handle)))
            self._plan = handle
            n = _lib.lib().cueq_b200_plan_table_bytes(handle)
            src = (C.c_char * n).from_address(_lib.lib().cueq_b200_plan_table_data(handle))
            self._tables_host = torch.frombuffer(bytearray(src), dtype=torch.uint8).clone()
        return self._plan

    def tables_on(self, device: torch.device) -> torch.Tensor:
        self.plan()
        t = self._tables_dev.get(device)
        if t is None:
            t = self._tables_host.to(device)
            self._tables_dev[device] = t
        return t

    def __del__(self):
        try:
            if self._plan is not None:
                _lib.lib().cueq_b200_plan_destroy(self._plan)
        except Exception:
            pass

    # -- derivatives -----------------------------------------------------------------------
    def derivative(self, requires_gradient: Tuple[bool, ...], has_cotangent: Tuple[bool, ...]) -> "Uniform1dProgram":
        key = (requires_gradient, has_cotangent)
        prog = self._derivatives.get(key)
        if prog is None:
            bwd = self.flat.backward(requires_gradient, has_cotangent)
            # gradient of input i takes the dtype of input i (same position in the new inputs)
            dmap = [i for i, r in enumerate(requires_gradient) if r]
            prog = Uniform1dProgram(bwd, self.math_dtype, dmap, name=self.name + "_bwd")
            if self._special is not None:
                prog._special = self._special.derive(requires_gradient, has_cotangent)
            if prog._special is None:
                attach_static(prog)
            self._derivatives[key] = prog
        return prog

    # -- launch ------------------------------------------------------------------------------
    def run(self, cfg: CallConfig, inputs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        device = inputs[0].device if inputs else None
        if device is None or device.type != "cuda":
            raise RuntimeError(
                "cuequivariance_b200 executes on CUDA devices only (there is no CPU fallback); "
                f"got tensors on {device}"
            )
        xs = []
        for i, (x, size) in enumerate(zip(inputs, self.row_sizes)):
            if x.ndim != 2 or x.shape[1] != size:
                raise ValueError(f"Input {i} has shape {tuple(x.shape)} but expected shape (*, {size}).")
            if x.shape[0] != cfg.inputs[i].rows:
                raise ValueError(f"Input {i} has {x.shape[0]} rows, the call was configured for {cfg.inputs[i].rows}.")
            xs.append(x.contiguous())
        outs = None
        if self._special is not None and cfg.batch > 0:
            outs = self._special.try_run(self, cfg, xs)
        if outs is None:
            from .transpose import transpose_blocks

            for i in range(self.num_inputs):
                if cfg.layout(i) is not None:
                    xs[i] = transpose_blocks(xs[i], cfg.layout(i), to_ir_mul=True)
            outs = [
                torch.zeros((spec.rows, self.row_sizes[self.num_inputs + j]), dtype=self.math_dtype, device=device)
                for j, spec in enumerate(cfg.outputs)
            ]
            if cfg.batch > 0:
                self._launch_generic(cfg, xs, outs, device)
            for j in range(self.num_outputs):
                lay = cfg.layout(self.num_inputs + j)
                if lay is not None:
                    outs[j] = transpose_blocks(outs[j], lay, to_ir_mul=False)
        result = []
        for j, o in enumerate(outs):
            m = self.output_dtype_map[j]
            want = self.math_dtype if m < 0 else inputs[m].dtype
            result.append(o if o.dtype == want else o.to(want))
        return result

    def _launch_generic(self, cfg: CallConfig, xs, outs, device):
        nb = self.num_inputs + self.num_outputs
        bufs = (_lib.Buffer * nb)()
        keep = []
        for b, (t, spec) in enumerate(zip(list(xs) + list(outs), cfg.inputs + cfg.outputs)):
            bufs[b].ptr = t.data_ptr() if t.numel() else None
            bufs[b].rows = spec.rows
            bufs[b].mode = spec.mode
            bufs[b].dtype = dtype_code(t.dtype)
            if spec.mode == _lib.INDEXED:
                idx = spec.index
                if idx.device != device:
                    raise ValueError("index tensors must live on the same device as the inputs")
                idx = idx.contiguous()
                keep.append(idx)
                bufs[b].index = idx.data_ptr() if idx.numel() else None
                bufs[b].index_is_64 = 1 if idx.dtype == torch.int64 else 0
            else:
                bufs[b].index = None
                bufs[b].index_is_64 = 0
        tables = self.tables_on(device)
        stream = torch.cuda.current_stream(device).cuda_stream
        from . import profiling

        with torch.cuda.device(device), profiling.kernel(f"u1d_generic[{self.name}]"):
            _lib.check(
                _lib.lib().cueq_b200_u1d_launch(self.plan(), tables.data_ptr(), cfg.batch, bufs, nb, C.c_void_p(stream))
            )


class StaticKernel:
    """Routes a program to the kernel generated for its polynomial at build time."""

    def __init__(self, kernel_id: int, name: str):
        self.kernel_id, self.name = kernel_id, name

    def try_run(self, program: "Uniform1dProgram", cfg: CallConfig, xs):
        from . import profiling

        if program.math_dtype != torch.float32 or any(x.dtype != torch.float32 for x in xs):
            return None
        if any(cfg.layout(b) is not None for b in range(program.num_inputs + program.num_outputs)):
            return None
        device = xs[0].device
        outs = [
            torch.zeros((spec.rows, program.row_sizes[program.num_inputs + j]), dtype=torch.float32, device=device)
            if spec.mode != _lib.BATCHED or program.buffer_dim[program.num_inputs + j] == 0
            else torch.empty((spec.rows, program.row_sizes[program.num_inputs + j]), dtype=torch.float32, device=device)
            for j, spec in enumerate(cfg.outputs)
        ]
        nb = program.num_inputs + program.num_outputs
        bufs = (_lib.Buffer * nb)()
        keep = []
        for b, (t, spec) in enumerate(zip(list(xs) + outs, cfg.inputs + cfg.outputs)):
            bufs[b].ptr = t.data_ptr() if t.numel() else None
            bufs[b].rows, bufs[b].mode, bufs[b].dtype = spec.rows, spec.mode, _lib.F32
            if spec.mode == _lib.INDEXED:
                idx = spec.index.contiguous()
                keep.append(idx)
                bufs[b].index = idx.data_ptr() if idx.numel() else None
                bufs[b].index_is_64 = 1 if idx.dtype == torch.int64 else 0
        stream = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
        with torch.cuda.device(device), profiling.kernel(f"u1d_static[{self.name}]"):
            _lib.check(_lib.lib().cueq_b200_u1d_static_launch(
                self.kernel_id, cfg.batch, program.extent, bufs, _lib.int32_array(program.buffer_dim),
                _lib.int32_array(program.buffer_num_segments), nb, stream))
        return outs

    def derive(self, requires_gradient, has_cotangent):
        return None  # the derivative program is matched by its own digest


SPLIT_STATIC_GRADIENTS = True   # one launch per gradient where each has a build-time kernel (see PolynomialFunction.backward)


def attach_static(program: "Uniform1dProgram") -> None:
    """Gives ``program`` the build-time kernel of its polynomial if the library has one."""
    from .static_poly import digest

    if program.math_dtype != torch.float32 or program._special is not None:
        return
    kid = _lib.lib().cueq_b200_u1d_static_find(digest(program.flat).encode())
    if kid >= 0:
        program._special = StaticKernel(kid, _lib.lib().cueq_b200_u1d_static_name(kid).decode())


def make_config(
    program: Uniform1dProgram,
    inputs: Sequence[torch.Tensor],
    input_indices: Dict[int, torch.Tensor],
    output_shapes: Dict[int, torch.Tensor],
    output_indices: Dict[int, torch.Tensor],
) -> Tuple[CallConfig, Dict[int, int]]:
    """Addressing modes of one forward call (reference rules:
    segmented_polynomial_uniform_1d.py:249-292, segmented_polynomial_naive.py:387-429).
    Returns the config and ``expand`` = {output j: rows} for one-row results that have to be
    broadcast afterwards."""
    batch = None

    def see(n: int, what: str):
        nonlocal batch
        if batch is None or batch == n:
            batch = n
        else:
            raise ValueError(f"inconsistent batch size: {what} has {n}, expected {batch}")

    in_specs = []
    for i, x in enumerate(inputs):
        if x.ndim == 0:
            raise ValueError(f"Input {i} has no dimensions")
        if i in input_indices:
            idx = input_indices[i]
            see(idx.shape[0], f"index of input {i}")
            in_specs.append(BufferSpec(_lib.INDEXED, x.shape[0], idx))
        elif x.shape[0] == 1:
            in_specs.append(BufferSpec(_lib.SHARED, 1, None))
        else:
            see(x.shape[0], f"input {i}")
            in_specs.append(BufferSpec(_lib.BATCHED, x.shape[0], None))
    for j, idx in output_indices.items():
        if j not in output_shapes:
            raise ValueError("output shapes must be provided for output indices")
        see(idx.shape[0], f"index of output {j}")
    if batch is None:  # every input is shared: one row is computed (and broadcast if asked)
        batch = 1
    out_specs, expand = [], {}
    for j in range(program.num_outputs):
        if j in output_indices:
            out_specs.append(BufferSpec(_lib.INDEXED, output_shapes[j].shape[0], output_indices[j]))
        elif j in output_shapes:
            rows = output_shapes[j].shape[0]
            if rows == batch and batch != 1:
                out_specs.append(BufferSpec(_lib.BATCHED, rows, None))
            elif rows == 1:
                out_specs.append(BufferSpec(_lib.SHARED, 1, None))
            elif batch == 1:
                out_specs.append(BufferSpec(_lib.SHARED, 1, None))
                expand[j] = rows
            else:
                raise ValueError(f"Input/output batch size mismatch ({rows}, ...) vs ({batch}, ...).")
        else:
            out_specs.append(BufferSpec(_lib.BATCHED if batch != 1 else _lib.SHARED, batch, None))
    return CallConfig(batch, tuple(in_specs), tuple(out_specs)), expand


def derivative_config(cfg: CallConfig, requires_gradient: Sequence[bool], has_cotangent: Sequence[bool]) -> CallConfig:
    """A cotangent is addressed like the output it belongs to, a gradient like its input."""
    ins = list(cfg.inputs) + [s for s, h in zip(cfg.outputs, has_cotangent) if h]
    outs = [s for s, r in zip(cfg.inputs, requires_gradient) if r]
    n_in = len(cfg.inputs)
    lay = [cfg.layout(b) for b in range(n_in + len(cfg.outputs))]
    lays = lay[:n_in] + [l for l, h in zip(lay[n_in:], has_cotangent) if h] + [l for l, r in zip(lay[:n_in], requires_gradient) if r]
    return CallConfig(cfg.batch, tuple(ins), tuple(outs), tuple(lays))


class PolynomialFunction(torch.autograd.Function):
    """``outputs = program(inputs)`` with ``backward`` = the derivative program, itself
    differentiable."""

    @staticmethod
    def forward(ctx, program: Uniform1dProgram, cfg: CallConfig, *inputs):
        ctx.program, ctx.cfg = program, cfg
        ctx.save_for_backward(*inputs)
        return tuple(program.run(cfg, [x.detach() for x in inputs]))

    @staticmethod
    def backward(ctx, *grad_outputs):
        program, cfg = ctx.program, ctx.cfg
        inputs = ctx.saved_tensors
        needs = tuple(bool(n) for n in ctx.needs_input_grad[2:])
        has = tuple(g is not None for g in grad_outputs)
        grads: List[Optional[torch.Tensor]] = [None] * len(inputs)
        if any(needs) and any(has):
            dprog = program.derivative(needs, has)
            cots = []
            for j, g in enumerate(grad_outputs):
                if g is not None:
                    cots.append(g.contiguous())
            # A build-time straight-line kernel that produces several gradients at once can need more registers
            # than a thread has (the symmetric contraction's weight + input gradient spills 0.8 KB per thread);
            # where every single gradient has a straight-line kernel of its own, one launch per gradient is faster.
            if SPLIT_STATIC_GRADIENTS and sum(needs) > 1 and isinstance(dprog._special, StaticKernel):
                singles = []
                for i, n in enumerate(needs):
                    if n:
                        one = tuple(k == i for k in range(len(needs)))
                        singles.append((i, one, program.derivative(one, has)))
                if all(isinstance(dp._special, StaticKernel) for _, _, dp in singles):
                    for i, one, dp in singles:
                        (grads[i],) = PolynomialFunction.apply(dp, derivative_config(cfg, one, has), *inputs, *cots)
                    return (None, None, *grads)
            dcfg = derivative_config(cfg, needs, has)
            res = PolynomialFunction.apply(dprog, dcfg, *inputs, *cots)
            it = iter(res)
            for i, n in enumerate(needs):
                if n:
                    grads[i] = next(it)
        return (None, None, *grads)


def evaluate(program: Uniform1dProgram, inputs, input_indices=None, output_shapes=None, output_indices=None, layouts=None):
    """``layouts``: optional {buffer id (inputs then outputs): ((mul, dim), ...)} for buffers
    held channel-major (mul_ir) by the caller."""
    input_indices = dict(input_indices or {})
    output_shapes = dict(output_shapes or {})
    output_indices = dict(output_indices or {})
    inputs = list(inputs)
    if len(inputs) != program.num_inputs:
        raise ValueError("the number of inputs must match the number of inputs of the polynomial")
    if _lib.CHECK_INDICES:
        input_indices = {k: _lib.checked_index(v, inputs[k].shape[0]) for k, v in input_indices.items()}
        output_indices = {k: _lib.checked_index(v, output_shapes[k] if isinstance(output_shapes[k], int) else output_shapes[k].shape[0])
                          for k, v in output_indices.items()}
    cfg, expand = make_config(program, inputs, input_indices, output_shapes, output_indices)
    if layouts:
        nb = program.num_inputs + program.num_outputs
        lays = []
        for b in range(nb):
            blocks = layouts.get(b)
            if blocks is not None and all(m == 1 or d == 1 for m, d in blocks):
                blocks = None  # both layouts coincide
            lays.append(None if blocks is None else tuple((int(m), int(d)) for m, d in blocks))
        if any(l is not None for l in lays):
            cfg = CallConfig(cfg.batch, cfg.inputs, cfg.outputs, tuple(lays))
    outs = list(PolynomialFunction.apply(program, cfg, *inputs))
    for j, rows in expand.items():
        outs[j] = outs[j].expand(rows, outs[j].shape[1]).clone()
    return outs
