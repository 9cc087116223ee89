"""Specialised execution of channelwise ("uvu") tensor products.

The polynomial ``uv,iu,jv,kuv+ijk`` (reference descriptor:
cuequivariance/group_theory/descriptors/irreps_tp.py:232-321) is split into *groups*: all
paths that read the same irrep of the first operand.  Each group runs as one launch of a
kernel whose Clebsch-Gordan arithmetic was written out at build time
(``csrc/gen_cw_groups.py``); gather of the first operand, the multiply-add and the
reduction over the edges of a receiver are fused, and layouts (mul_ir / ir_mul) are
handled in the addressing.  This module holds the pattern functions shared by the code
generator and the run-time matcher, and the matcher itself.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

from .cg import so3_clebsch_gordan


# ---- patterns shared with the code generator ---------------------------------------------
def pair_pattern(l1: int, l2: int, l3: int, major: str) -> List[Tuple[int, int, List[Tuple[int, float]]]]:
    """Non-zero ``(i, k)`` pairs of the coupling tensor of (l1, l2, l3) with their ``(j, C)``
    terms; ``major='k'`` orders pairs by k then i (forward), ``'i'`` by i then k (backward)."""
    c = so3_clebsch_gordan(l1, l2, l3)[0]
    d1, d2, d3 = c.shape
    order = [(i, k) for k in range(d3) for i in range(d1)] if major == "k" else [(i, k) for i in range(d1) for k in range(d3)]
    out = []
    for i, k in order:
        js = [j for j in range(d2) if c[i, j, k] != 0.0]
        if js:
            out.append((i, k, [(j, float(c[i, j, k])) for j in js]))
    return out


def value_pattern(l1: int, l2: int, l3: int):
    """The distinct values among the entries ``M[i, k] = sum_j C[i, j, k] x2[j]`` of a coupling, up to sign.

    Many (i, k) pairs carry the same linear combination of x2 (or its negative): for l <= 3 there are 207
    distinct ones among 311 pairs.  Returns ``(values, pairs)``: ``values[s]`` = the ``(j, coefficient)`` terms of
    slot ``s`` (first coefficient positive), ``pairs`` = ``(i, k, slot, sign)`` in k-major order with
    ``M[i, k] = sign * value[slot]``.  The forward kernels broadcast the values instead of the pairs."""
    values, index, pairs = [], {}, []
    for i, k, terms in pair_pattern(l1, l2, l3, "k"):
        t = sorted(terms)
        sign = 1.0 if t[0][1] > 0 else -1.0
        key = tuple((j, round(sign * c, 12)) for j, c in t)
        s = index.get(key)
        if s is None:
            s = index[key] = len(values)
            values.append([(j, sign * c) for j, c in t])
        pairs.append((i, k, s, sign))
    return values, pairs


SPLIT_GROUPS = False  # measured on B200: one launch per irrep beats two lighter launches


def split_group(l1: int, paths: Sequence[Tuple[int, int]]) -> List[List[Tuple[int, int]]]:
    """How the paths that read irrep ``l1`` are divided into kernel launches.  A launch keeps
    one accumulator per output component of its paths in registers, so large groups are cut
    in two parts of similar arithmetic weight (the two heaviest couplings form one part);
    this keeps four channels per thread within the register budget."""
    paths = list(paths)
    if not SPLIT_GROUPS or (len(paths) <= 4 and sum(2 * l3 + 1 for _, l3 in paths) <= 16):
        return [paths]
    weight = {p: len(pair_pattern(l1, p[0], p[1], "k")) for p in paths}
    heavy = sorted(paths, key=lambda p: -weight[p])[:2]
    light = [p for p in paths if p not in heavy]
    return [light, [p for p in paths if p in heavy]]


def group_signature(l1: int, paths: Sequence[Tuple[int, int]]) -> str:
    return f"{l1}:" + ",".join(f"{a}.{b}" for a, b in paths)


# ---- run-time side ----------------------------------------------------------------------------
class _CsrCache:
    """Receiver index -> (order or None, rowptr).  Keyed on the tensor's storage address and
    version counter, so in-place updates of the index are noticed; the cache holds a
    reference to the tensor, which keeps that address from being recycled."""

    def __init__(self, capacity: int = 8):
        self.capacity = capacity
        self.entries: list = []

    def get(self, index, num_rows: int):
        import torch

        key = (index.data_ptr(), index.numel(), index.dtype, index._version, num_rows, index.device)
        for k, ref, val in self.entries:
            if k == key and ref is index:
                return val
        idx = index if index.dtype == torch.int32 else index.to(torch.int32)
        if idx.numel() > 1 and not bool((idx[1:] >= idx[:-1]).all()):
            sorted_idx, order = torch.sort(idx, stable=True)
            order = order.to(torch.int32)
        else:
            sorted_idx, order = idx, None
        bounds = torch.arange(num_rows + 1, device=index.device, dtype=torch.int32)
        rowptr = torch.searchsorted(sorted_idx.contiguous(), bounds, right=False).to(torch.int32)
        val = (order, rowptr)
        self.entries.append((key, index, val))
        if len(self.entries) > self.capacity:
            self.entries.pop(0)
        return val

    def get_passes(self, receivers, senders, num_rows: int, num_senders: int, passes: int):
        """CSR over (pass, receiver) rows, pass = which of ``passes`` equal ranges the sender
        falls in: edges are visited pass by pass, so that only 1/passes of the node rows is
        gathered from / reduced into at a time (keeps that working set inside L2)."""
        import torch

        key = ("passes", receivers.data_ptr(), receivers._version, senders.data_ptr(), senders._version, num_rows, num_senders, passes)
        for k, ref, val in self.entries:
            if k == key and ref is receivers:
                return val
        span = (num_senders + passes - 1) // passes
        rows = (senders.to(torch.int64) // span) * num_rows + receivers.to(torch.int64)
        sorted_rows, order = torch.sort(rows, stable=True)
        bounds = torch.arange(passes * num_rows + 1, device=receivers.device, dtype=torch.int64)
        rowptr = torch.searchsorted(sorted_rows.contiguous(), bounds, right=False).to(torch.int32)
        val = (order.to(torch.int32), rowptr)
        self.entries.append((key, receivers, val))
        if len(self.entries) > self.capacity:
            self.entries.pop(0)
        return val

    def int32(self, index):
        import torch

        if index.dtype == torch.int32:
            return index.contiguous()
        key = ("i32", index.data_ptr(), index.numel(), index._version, index.device)
        for k, ref, val in self.entries:
            if k == key and ref is index:
                return val
        val = index.to(torch.int32).contiguous()
        self.entries.append((key, index, val))
        if len(self.entries) > self.capacity:
            self.entries.pop(0)
        return val


_CSR = _CsrCache()
SENDER_PASSES = 1  # backward: visit the edges in this many sender-range passes when the node table exceeds 64 MB
STAGING = 0  # forward kernels: 0 = per-lane cp.async staging, 1 = bulk copies (TMA) signalled on an mbarrier
CHANNELS_PER_LANE = 0  # 0: the library chooses; 2 or 4 force a variant (used by the tests)
BWD_VARIANT = 0  # backward kernels: 0 = the library chooses, 1 = one warp per receiver, 2 = one thread block per receiver, 3 = 2 with bulk reductions of the x1 gradient
_IDENTITY_ROWPTR: dict = {}


def _library_groups() -> dict:
    from . import _lib

    L = _lib.lib()
    return {L.cueq_b200_cw_group_signature(g).decode(): g for g in range(L.cueq_b200_cw_num_groups())}


class ChannelwisePlan:
    """What the kernels need for one channelwise polynomial: per group the library kernel
    id, segment offsets and the M-tables (forward: k-major pairs, backward: i-major)."""

    def __init__(self, groups, extent, row_sizes, x1_blocks, out_blocks):
        self.groups = groups
        self.extent = extent
        self.row_sizes = row_sizes          # (w, x1, x2, out) elements per row
        self.x1_blocks = x1_blocks          # ((mul, dim), ...) of x1
        self.out_blocks = out_blocks
        self._dev: dict = {}

    def tables_on(self, device):
        import torch

        t = self._dev.get(device)
        if t is None:
            t = []
            for g in self.groups:
                t.append({
                    k: (torch.tensor(g[k][0], dtype=torch.int32, device=device),
                        torch.tensor(g[k][1], dtype=torch.int32, device=device),
                        torch.tensor(g[k][2], dtype=torch.float32, device=device))
                    for k in ("fwd_tab", "bwd_tab")
                })
            self._dev[device] = t
        return t


def match_channelwise(polynomial) -> Optional[ChannelwisePlan]:
    """Recognises ``uv,iu,jv,kuv+ijk`` built from SO(3)/O(3) coupling tensors whose groups all
    have a kernel in the library; returns None otherwise."""
    if len(polynomial.operations) != 1 or polynomial.num_inputs != 3 or polynomial.num_outputs != 1:
        return None
    ope, d = polynomial.operations[0]
    if d.subscripts != "uv,iu,jv,kuv+ijk" or tuple(ope.buffers) != (0, 1, 2, 3):
        return None
    w_op, x1_op, x2_op, out_op = d.operands
    if not x1_op.segments or not x2_op.segments:
        return None
    extent = x1_op.segments[0][1]
    if extent % 4 or any(s[1] != extent for s in x1_op.segments) or any(s[1] != 1 for s in x2_op.segments):
        return None
    if any(s[0] % 2 == 0 for s in x1_op.segments + x2_op.segments):
        return None
    l2s = [(s[0] - 1) // 2 for s in x2_op.segments]
    if l2s != list(range(len(l2s))):
        return None  # x2 must be one copy of l = 0, 1, 2, ... in order
    x2_off = x2_op.offsets()
    w_off, x1_off, out_off = w_op.offsets(), x1_op.offsets(), out_op.offsets()
    by_i1: dict = {}
    seen_w, seen_o = set(), set()
    for path in d.paths:
        sw, s1, s2, so = path.indices
        c = path.coefficients
        d1, d2, d3 = c.shape
        if d3 % 2 == 0 or w_op.segments[sw] != (extent, 1) or out_op.segments[so] != (d3, extent, 1):
            return None
        if sw in seen_w or so in seen_o:
            return None
        seen_w.add(sw)
        seen_o.add(so)
        l1, l2, l3 = (d1 - 1) // 2, (d2 - 1) // 2, (d3 - 1) // 2
        ref = so3_clebsch_gordan(l1, l2, l3)
        if ref.shape[0] != 1:
            return None
        ref = ref[0]
        nz = ref != 0
        if not np.array_equal(nz, c != 0):
            return None
        alpha = float((c[nz] / ref[nz]).mean())
        if not np.allclose(c, alpha * ref, rtol=1e-12, atol=1e-14):
            return None
        by_i1.setdefault(s1, []).append((l1, l2, l3, sw, so, c))
    lib = _library_groups()
    groups = []
    launches = []
    for s1, plist in sorted(by_i1.items()):
        l1 = plist[0][0]
        all_paths = [(l2, l3) for _, l2, l3, _, _, _ in plist]
        if len(set(all_paths)) != len(all_paths):
            return None
        parts = split_group(l1, all_paths)
        if any(group_signature(l1, part) not in lib for part in parts):
            parts = [all_paths]
        for part in parts:
            launches.append((s1, [p for p in plist if (p[1], p[2]) in part]))
    for s1, plist in launches:
        l1 = plist[0][0]
        sig = group_signature(l1, [(l2, l3) for _, l2, l3, _, _, _ in plist])
        if sig not in lib:
            return None
        g = {"id": lib[sig], "x1_off": x1_off[s1], "w_off": [w_off[p[3]] for p in plist],
             "out_off": [out_off[p[4]] for p in plist], "npath": len(plist), "out_segs": [p[4] for p in plist],
             "x1_width": x1_op.segments[s1][0] * x1_op.segments[s1][1], "l1": l1}
        # backward: one table entry per non-zero (i, k) pair, i-major
        start, tj, tc = [0], [], []
        for l1_, l2, l3, _, _, c in plist:
            for i, k, terms in pair_pattern(l1_, l2, l3, "i"):
                for j, _ref in terms:
                    tj.append(x2_off[l2] + j)
                    tc.append(float(c[i, j, k]))
                start.append(len(tj))
        g["bwd_tab"] = (start, tj, tc)
        # forward: one entry per distinct value (see value_pattern); the descriptor's coefficient of a value is
        # read off the first pair that carries it
        start, tj, tc = [0], [], []
        for l1_, l2, l3, _, _, c in plist:
            values, pairs = value_pattern(l1_, l2, l3)
            first = {}
            for i, k, s, sign in pairs:
                first.setdefault(s, (i, k, sign))
            for s, terms in enumerate(values):
                i, k, sign = first[s]
                for j, _ref in terms:
                    tj.append(x2_off[l2] + j)
                    tc.append(sign * float(c[i, j, k]))
                start.append(len(tj))
        g["fwd_tab"] = (start, tj, tc)
        g["nterm"] = len(g["bwd_tab"][1])
        g["nterm_fwd"] = len(g["fwd_tab"][1])
        groups.append(g)
    # every output segment must be produced by exactly one path (else rows would be incomplete)
    if len(seen_o) != out_op.num_segments:
        return None
    x1_blocks = tuple((s[1], s[0]) for s in x1_op.segments)
    out_blocks = tuple((s[1] * s[2], s[0]) for s in out_op.segments)
    return ChannelwisePlan(groups, extent, (w_op.size, x1_op.size, x2_op.size, out_op.size), x1_blocks, out_blocks)


def _is_mul_ir(layout, blocks) -> Optional[bool]:
    """None if ``layout`` is something the kernels do not understand."""
    if layout is None:
        return False
    return True if tuple(layout) == tuple(blocks) else None


class _ChannelwiseBase:
    def __init__(self, plan: ChannelwisePlan):
        self.plan = plan

    def _common(self, program, cfg, xs, n_in):
        import torch

        from . import _lib

        plan = self.plan
        if program.math_dtype != torch.float32 or any(x.dtype != torch.float32 for x in xs):
            return None
        w_s, x1_s, x2_s = cfg.inputs[0], cfg.inputs[1], cfg.inputs[2]
        if w_s.mode != _lib.BATCHED or x2_s.mode != _lib.BATCHED or x1_s.mode == _lib.SHARED:
            return None
        if cfg.layout(0) is not None or cfg.layout(2) is not None:
            return None
        x1_mul_ir = _is_mul_ir(cfg.layout(1), plan.x1_blocks)
        if x1_mul_ir is None or any(x.data_ptr() % 16 for x in xs):
            return None
        senders = _CSR.int32(x1_s.index) if x1_s.mode == _lib.INDEXED else None
        recv_spec = cfg.inputs[3] if n_in >= 4 else cfg.outputs[0]
        receivers = recv_spec.index if recv_spec.mode == _lib.INDEXED else None
        return dict(x1_mul_ir=x1_mul_ir, senders=senders, receivers=receivers)

    def _csr(self, spec, batch, device):
        import torch

        from . import _lib

        if spec.mode == _lib.INDEXED:
            order, rowptr = _CSR.get(spec.index, spec.rows)
            return order, rowptr, spec.rows
        if spec.mode == _lib.BATCHED:
            key = (batch, device)
            rp = _IDENTITY_ROWPTR.get(key)
            if rp is None:
                rp = torch.arange(batch + 1, dtype=torch.int32, device=device)
                _IDENTITY_ROWPTR.clear()
                _IDENTITY_ROWPTR[key] = rp
            return None, rp, batch
        return None

    def _args(self, g, tabs, which, common, order, rowptr, nrecv, out_mul_ir, tensors, x1_is_block=False):
        """``x1_is_block``: tensors['x1'] (and 'gx1') hold only this group's irrep block,
        ``[rows, extent * d1]`` (unit stride along the row, any row stride), instead of full rows.  The constant part of the
        argument block is built once per (group, direction) and copied."""
        import ctypes as C

        from . import _lib

        plan = self.plan
        cache = g.setdefault("_arg_templates", {})
        tmpl = cache.get(which)
        if tmpl is None:
            t = _lib.CwArgs()
            t.w_stride, t.x1_stride, t.x2_stride, t.out_stride = plan.row_sizes
            t.extent = plan.extent
            t.x1_offset = g["x1_off"]
            t.num_paths = g["npath"]
            t.num_terms = g["nterm"] if which == "bwd_tab" else g["nterm_fwd"]
            for q in range(g["npath"]):
                t.w_offset[q] = g["w_off"][q]
                t.out_offset[q] = g["out_off"][q]
            keep = None
            if which == "bwd_tab":
                keep = (C.c_float * g["nterm"])(*g["bwd_tab"][2])
                t.bwd_coef = C.cast(keep, C.POINTER(C.c_float))
            tmpl = (bytes(t), keep)
            cache[which] = tmpl
        a = _lib.CwArgs.from_buffer_copy(tmpl[0])
        for k, t in tensors.items():
            if t is not None and t.numel():
                setattr(a, k, t.data_ptr())
        if common["senders"] is not None:
            a.senders = common["senders"].data_ptr()
        if order is not None:
            a.order = order.data_ptr()
        a.rowptr = rowptr.data_ptr()
        ts, tj, tc = tabs[which]
        a.tab_start, a.tab_j, a.tab_c = ts.data_ptr(), tj.data_ptr(), tc.data_ptr()
        a.num_receivers = nrecv
        if x1_is_block:
            # may be a column slice of a wider tensor (several irrep blocks gathered together); a
            # gradient block, if any, must then be the matching slice of an equally wide tensor
            a.x1_stride = tensors["x1"].stride(0)
            a.x1_offset = 0
            gx1 = tensors.get("gx1")
            if gx1 is not None and gx1.stride(0) != a.x1_stride:
                raise ValueError("channelwise: the x1 block and its gradient block must have the same row stride")
        a.x1_mul_ir = 1 if common["x1_mul_ir"] else 0
        a.out_mul_ir = 1 if out_mul_ir else 0
        # the scalar-x1 group is the one where four channels per lane fit the register budget and pay off
        # (config 3: forward 0.58 -> 0.46 ms, backward 1.15 -> 1.00 ms; every other group is slower with four)
        a.channels_per_lane = CHANNELS_PER_LANE or (4 if g.get("l1") == 0 and plan.extent % 128 == 0 else 0)
        a.staging = STAGING if which == "fwd_tab" else 0
        a.variant = BWD_VARIANT if which == "bwd_tab" else 0
        if a.staging:
            a.status = _lib.status_word(tensors["w"].device).data_ptr()
        return a, tmpl[1]

    # -- kernel launches shared by the first- and second-order handlers ------------------------
    def launch_forward_group(self, gi, common, csr, mul_ir, w, x1_block, x2, out):
        """One group of the forward pass with that group's x1 block given separately (used by
        the multi-GPU path, where blocks arrive one by one)."""
        import ctypes as C

        import torch

        from . import _lib, profiling

        order, rowptr, nrecv = csr
        g, t = self.plan.groups[gi], self.plan.tables_on(w.device)[gi]
        stream = C.c_void_p(torch.cuda.current_stream(w.device).cuda_stream)
        with torch.cuda.device(w.device):
            a, _ = self._args(g, t, "fwd_tab", common, order, rowptr, nrecv, mul_ir, dict(w=w, x1=x1_block, x2=x2, out=out), x1_is_block=True)
            with profiling.kernel(f"cw_fwd[{g['id']}]", stream):
                _lib.check(_lib.lib().cueq_b200_cw_forward(g["id"], C.byref(a), stream))

    def launch_backward_group(self, gi, common, csr, mul_ir, w, x1_block, x2, gout, gw, gx1_block, gx2):
        import ctypes as C

        import torch

        from . import _lib, profiling

        order, rowptr, nrecv = csr
        g, t = self.plan.groups[gi], self.plan.tables_on(w.device)[gi]
        stream = C.c_void_p(torch.cuda.current_stream(w.device).cuda_stream)
        with torch.cuda.device(w.device):
            a, keep = self._args(g, t, "bwd_tab", common, order, rowptr, nrecv, mul_ir,
                                 dict(w=w, x1=x1_block, x2=x2, gout=gout, gw=gw, gx1=gx1_block, gx2=gx2), x1_is_block=True)
            with profiling.kernel(f"cw_bwd[{g['id']}]", stream):
                _lib.check(_lib.lib().cueq_b200_cw_backward(g["id"], C.byref(a), stream))
            del keep

    def _launch_forward(self, common, csr, mul_ir, w, x1, x2):
        import ctypes as C

        import torch

        from . import _lib, profiling

        plan = self.plan
        order, rowptr, nrecv = csr
        out = torch.empty((nrecv, plan.row_sizes[3]), dtype=torch.float32, device=w.device)
        tabs = plan.tables_on(w.device)
        stream = C.c_void_p(torch.cuda.current_stream(w.device).cuda_stream)
        with torch.cuda.device(w.device):
            for g, t in zip(plan.groups, tabs):
                a, _ = self._args(g, t, "fwd_tab", common, order, rowptr, nrecv, mul_ir, dict(w=w, x1=x1, x2=x2, out=out))
                with profiling.kernel(f"cw_fwd[{g['id']}]", stream):
                    _lib.check(_lib.lib().cueq_b200_cw_forward(g["id"], C.byref(a), stream))
        return out

    def _launch_backward(self, common, csr, mul_ir, w, x1, x2, gout, needs):
        import ctypes as C

        import torch

        from . import _lib, profiling

        plan = self.plan
        order, rowptr, nrecv = csr
        recv_mod = 0
        if (needs[1] and SENDER_PASSES > 1 and common["senders"] is not None and common.get("receivers") is not None
                and x1.shape[0] * plan.row_sizes[1] * 4 > (64 << 20)):
            order, rowptr = _CSR.get_passes(common["receivers"], common["senders"], nrecv, x1.shape[0], SENDER_PASSES)
            recv_mod, nrecv = nrecv, nrecv * SENDER_PASSES
        dev = w.device
        gw = torch.empty_like(w) if needs[0] else None
        gx1 = torch.zeros_like(x1) if needs[1] else None
        gx2 = torch.zeros_like(x2) if needs[2] else None
        tabs = plan.tables_on(dev)
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            for g, t in zip(plan.groups, tabs):
                a, keep = self._args(g, t, "bwd_tab", common, order, rowptr, nrecv, mul_ir,
                                     dict(w=w, x1=x1, x2=x2, gout=gout, gw=gw, gx1=gx1, gx2=gx2))
                a.recv_mod = recv_mod
                with profiling.kernel(f"cw_bwd[{g['id']}]", stream):
                    _lib.check(_lib.lib().cueq_b200_cw_backward(g["id"], C.byref(a), stream))
                del keep
        return gw, gx1, gx2


class ChannelwiseForward(_ChannelwiseBase):
    """``try_run`` returns the outputs, or None when the call is outside what the kernels
    cover (the generic executor then takes it)."""

    def try_run(self, program, cfg, xs):
        common = self._common(program, cfg, xs, 3)
        if common is None:
            return None
        out_mul_ir = _is_mul_ir(cfg.layout(3), self.plan.out_blocks)
        csr = self._csr(cfg.outputs[0], cfg.batch, xs[0].device)
        if out_mul_ir is None or csr is None or out_mul_ir != common["x1_mul_ir"]:
            return None
        return [self._launch_forward(common, csr, out_mul_ir, *xs)]

    def derive(self, requires_gradient, has_cotangent):
        if not has_cotangent[0]:
            return None
        return ChannelwiseBackward(self.plan, tuple(requires_gradient))


class ChannelwiseBackward(_ChannelwiseBase):
    """Inputs (w, x1, x2, gout) -> gradients of the flagged inputs."""

    def __init__(self, plan, needs):
        super().__init__(plan)
        self.needs = needs

    def _check(self, program, cfg, xs, n_in, grad_specs):
        """Common admission test; ``grad_specs`` = [(output position, input it mirrors)]."""
        common = self._common(program, cfg, xs, n_in)
        if common is None:
            return None
        out_mul_ir = _is_mul_ir(cfg.layout(3), self.plan.out_blocks)
        csr = self._csr(cfg.inputs[3], cfg.batch, xs[0].device)
        if out_mul_ir is None or csr is None or out_mul_ir != common["x1_mul_ir"]:
            return None
        for k, i in grad_specs:  # gradient layouts and addressing must mirror their inputs
            if cfg.layout(n_in + k) != cfg.layout(i) or cfg.outputs[k].mode != cfg.inputs[i].mode:
                return None
            if cfg.outputs[k].index is not cfg.inputs[i].index:
                return None
        return common, csr, out_mul_ir

    def try_run(self, program, cfg, xs):
        wanted = [i for i, n in enumerate(self.needs) if n]
        ok = self._check(program, cfg, xs, 4, list(enumerate(wanted)))
        if ok is None:
            return None
        common, csr, mul_ir = ok
        res = self._launch_backward(common, csr, mul_ir, *xs, self.needs)
        return [t for t, need in zip(res, self.needs) if need]

    def derive(self, requires_gradient, has_cotangent):
        return ChannelwiseSecondOrder(self.plan, self.needs, tuple(requires_gradient), tuple(has_cotangent))


class ChannelwiseSecondOrder(ChannelwiseBackward):
    """Derivative of the backward call, composed from the same first-order kernels.

    With T(w, x1, x2, g) = <g, F(w, x1, x2)> linear in each argument, the backward call
    returns the partial derivatives of T; pairing them with cotangents (tw, tx1, tx2) gives
    L = T(tw, x1, x2, g) + T(w, tx1, x2, g) + T(w, x1, tx2, g), whose gradients are again
    forward and backward evaluations with one argument replaced by a cotangent:
        dL/dg  = F(tw, x1, x2) + F(w, tx1, x2) + F(w, x1, tx2)
        dL/dw  = f_w(tx1, x2, g) + f_w(x1, tx2, g)       (f_w does not depend on w)
        dL/dx1 = f_x1(tw, x2, g) + f_x1(w, tx2, g)
        dL/dx2 = f_x2(tw, x1, g) + f_x2(w, tx1, g)
    Inputs (w, x1, x2, g, cotangents of the first-order outputs that have one); outputs the
    gradients of the flagged inputs among (w, x1, x2, g)."""

    def __init__(self, plan, first_needs, requires_gradient, has_cotangent):
        super().__init__(plan, first_needs)
        self.req = requires_gradient
        self.has = has_cotangent

    def try_run(self, program, cfg, xs):
        import torch

        first_outputs = [i for i, n in enumerate(self.needs) if n]           # which of (gw, gx1, gx2) exist
        cots = {}
        k = 4
        for pos, i in enumerate(first_outputs):
            if self.has[pos]:
                cots[i] = k
                k += 1
        n_in = k
        if len(xs) != n_in or len(self.req) != 4:
            return None
        # cotangents must be addressed like the inputs they pair with
        for i, b in cots.items():
            if cfg.layout(b) != cfg.layout(i) or cfg.inputs[b].mode != cfg.inputs[i].mode or cfg.inputs[b].index is not cfg.inputs[i].index:
                return None
        wanted = [i for i, r in enumerate(self.req) if r]
        ok = self._check(program, cfg, xs, n_in, list(enumerate(wanted)))
        if ok is None:
            return None
        common, csr, mul_ir = ok
        w, x1, x2, g = xs[:4]
        tw, tx1, tx2 = (xs[cots[i]] if i in cots else None for i in range(3))
        out = {0: None, 1: None, 2: None, 3: None}

        def add(i, t):
            if t is not None:
                out[i] = t if out[i] is None else out[i] + t

        if self.req[3]:
            for a, b, c in ((tw, x1, x2), (w, tx1, x2), (w, x1, tx2)):
                if a is not None and b is not None and c is not None:
                    add(3, self._launch_forward(common, csr, mul_ir, a, b, c))
        if tx1 is not None and (self.req[0] or self.req[2]):
            gw_, _, gx2_ = self._launch_backward(common, csr, mul_ir, w, tx1, x2, g, (self.req[0], False, self.req[2]))
            add(0, gw_), add(2, gx2_)
        if tx2 is not None and (self.req[0] or self.req[1]):
            gw_, gx1_, _ = self._launch_backward(common, csr, mul_ir, w, x1, tx2, g, (self.req[0], self.req[1], False))
            add(0, gw_), add(1, gx1_)
        if tw is not None and (self.req[1] or self.req[2]):
            _, gx1_, gx2_ = self._launch_backward(common, csr, mul_ir, tw, x1, x2, g, (False, self.req[1], self.req[2]))
            add(1, gx1_), add(2, gx2_)
        res = []
        for i in wanted:
            if out[i] is None:
                ref = (w, x1, x2, g)[i]
                out[i] = torch.zeros_like(ref)
            res.append(out[i])
        return res

    def derive(self, requires_gradient, has_cotangent):
        return None  # third derivatives run on the generic executor


def attach_specialisation(program) -> None:
    """Routes a matching program to the channelwise kernels (float32 math only)."""
    import torch

    if program.math_dtype != torch.float32:
        return
    plan = match_channelwise(program.original)
    if plan is not None:
        program._special = ChannelwiseForward(plan)
