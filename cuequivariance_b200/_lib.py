"""ctypes binding of ``libcueq_b200.so`` (declarations mirror ``include/cueq_b200.h``).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libcueq_b200.so"

F32, F64, BF16, F16 = 0, 1, 2, 3
SHARED, BATCHED, INDEXED = 0, 1, 2
MAX_BUFFERS, MAX_OPERANDS = 16, 8


class U1dDesc(C.Structure):
    _fields_ = [
        ("operand_extent", C.c_int32),
        ("num_inputs", C.c_int32),
        ("num_outputs", C.c_int32),
        ("buffer_dim", C.POINTER(C.c_int32)),
        ("buffer_num_segments", C.POINTER(C.c_int32)),
        ("num_operations", C.c_int32),
        ("num_operands", C.POINTER(C.c_int32)),
        ("operations", C.POINTER(C.c_int32)),
        ("num_paths", C.POINTER(C.c_int32)),
        ("path_indices", C.POINTER(C.c_int32)),
        ("path_coefficients", C.POINTER(C.c_double)),
        ("math_dtype", C.c_int32),
    ]


class Buffer(C.Structure):
    _fields_ = [
        ("ptr", C.c_void_p),
        ("rows", C.c_int64),
        ("mode", C.c_int32),
        ("dtype", C.c_int32),
        ("index", C.c_void_p),
        ("index_is_64", C.c_int32),
        ("reserved", C.c_int32),
    ]


class CwArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("x1", C.c_void_p), ("x2", C.c_void_p), ("out", C.c_void_p),
        ("gout", C.c_void_p), ("gw", C.c_void_p), ("gx1", C.c_void_p), ("gx2", C.c_void_p),
        ("senders", C.c_void_p), ("order", C.c_void_p), ("rowptr", C.c_void_p),
        ("tab_start", C.c_void_p), ("tab_j", C.c_void_p), ("tab_c", C.c_void_p),
        ("bwd_coef", C.POINTER(C.c_float)),
        ("w_stride", C.c_int64), ("x1_stride", C.c_int64), ("x2_stride", C.c_int64), ("out_stride", C.c_int64),
        ("num_receivers", C.c_int64),
        ("extent", C.c_int32), ("x1_offset", C.c_int32), ("num_paths", C.c_int32), ("num_terms", C.c_int32),
        ("w_offset", C.c_int32 * 8), ("out_offset", C.c_int32 * 8),
        ("x1_mul_ir", C.c_int32), ("out_mul_ir", C.c_int32), ("channels_per_lane", C.c_int32), ("staging", C.c_int32),
        ("status", C.c_void_p), ("recv_mod", C.c_int32), ("variant", C.c_int32),
    ]


class CwNoAllocArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("x1", C.c_void_p), ("x2", C.c_void_p), ("out", C.c_void_p),
        ("senders", C.c_void_p), ("receivers", C.c_void_p),
        ("tab_start_host", C.POINTER(C.c_int32)), ("tab_j_host", C.POINTER(C.c_int32)), ("tab_c_host", C.POINTER(C.c_float)),
        ("w_stride", C.c_int64), ("x1_stride", C.c_int64), ("x2_stride", C.c_int64), ("out_stride", C.c_int64),
        ("num_edges", C.c_int64), ("num_receivers", C.c_int64),
        ("extent", C.c_int32), ("x1_offset", C.c_int32), ("num_paths", C.c_int32), ("num_terms", C.c_int32),
        ("w_offset", C.c_int32 * 8), ("out_offset", C.c_int32 * 8),
        ("mul_ir", C.c_int32), ("reserved", C.c_int32),
    ]


class PushArgs(C.Structure):
    _fields_ = [("dst", C.c_void_p * 8), ("src", C.c_void_p * 8), ("bytes", C.c_int64 * 8), ("num_pieces", C.c_int32), ("blocks_per_piece", C.c_int32)]


class ShArgs(C.Structure):
    _fields_ = [
        ("vec", C.c_void_p), ("y", C.c_void_p), ("gvec", C.c_void_p),
        ("rows", C.c_int64), ("ld_vec", C.c_int64), ("ld_y", C.c_int64), ("ld_gvec", C.c_int64),
        ("ls_mask", C.c_uint32), ("normalize", C.c_int32), ("dtype", C.c_int32), ("reserved", C.c_int32),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("group_stride", C.c_int64),
        ("rows_per_group", C.c_int32), ("accumulate", C.c_int32), ("out_bf16", C.c_int32),
        ("a_mn_major", C.c_int32), ("b_mn_major", C.c_int32), ("c_is_zero", C.c_int32),
        ("status", C.c_void_p),
    ]


class FctpArgs(C.Structure):
    _fields_ = [
        ("x1", C.c_void_p), ("x2", C.c_void_p), ("z", C.c_void_p), ("gx1", C.c_void_p), ("gx2", C.c_void_p),
        ("cg", C.POINTER(C.c_float)),
        ("ld1", C.c_int64), ("ld2", C.c_int64), ("batch", C.c_int64),
        ("off1", C.c_int32), ("off2", C.c_int32),
        ("d1", C.c_int32), ("d2", C.c_int32), ("d3", C.c_int32), ("U", C.c_int32), ("V", C.c_int32),
        ("x_dtype", C.c_int32), ("z_dtype", C.c_int32), ("ldz", C.c_int32),
    ]


class FctpFusedPath(C.Structure):
    _fields_ = [
        ("off1", C.c_int32), ("off2", C.c_int32), ("d1", C.c_int32), ("d2", C.c_int32),
        ("w_row0", C.c_int32), ("reserved", C.c_int32), ("c", C.c_float * 25), ("reserved2", C.c_float),
    ]


class FctpFusedTask(C.Structure):
    _fields_ = [("out_off", C.c_int32), ("num_paths", C.c_int32), ("paths", FctpFusedPath * 4)]


class FctpFusedArgs(C.Structure):
    _fields_ = [
        ("x1", C.c_void_p), ("x2", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p),
        ("ld1", C.c_int64), ("ld2", C.c_int64), ("ldo", C.c_int64), ("batch", C.c_int64), ("w_rows", C.c_int64),
        ("out_dtype", C.c_int32), ("num_tasks", C.c_int32),
        ("tasks", C.POINTER(FctpFusedTask)), ("status", C.c_void_p),
    ]


class FctpFusedUnit(C.Structure):
    _fields_ = [
        ("offa", C.c_int32), ("offb", C.c_int32), ("da", C.c_int32), ("db", C.c_int32),
        ("w_row0", C.c_int32), ("nk", C.c_int32), ("goff", C.c_int32 * 2), ("c", (C.c_float * 25) * 2),
    ]


class FctpFusedGxArgs(C.Structure):
    _fields_ = [
        ("xb", C.c_void_p), ("gout", C.c_void_p), ("w", C.c_void_p), ("gxa", C.c_void_p),
        ("ldb", C.c_int64), ("ldg", C.c_int64), ("lda", C.c_int64), ("batch", C.c_int64), ("w_rows", C.c_int64),
        ("num_units", C.c_int32), ("reserved", C.c_int32),
        ("units", C.POINTER(FctpFusedUnit)), ("status", C.c_void_p),
    ]


class FctpFusedWUnit(C.Structure):
    _fields_ = [
        ("off1", C.c_int32), ("off2", C.c_int32), ("d1", C.c_int32), ("d2", C.c_int32),
        ("w_row0", C.c_int32), ("goff", C.c_int32), ("c", C.c_float * 25), ("reserved", C.c_float),
    ]


class FctpFusedGwArgs(C.Structure):
    _fields_ = [
        ("x1", C.c_void_p), ("x2", C.c_void_p), ("gout", C.c_void_p), ("gw", C.c_void_p),
        ("ld1", C.c_int64), ("ld2", C.c_int64), ("ldg", C.c_int64), ("batch", C.c_int64), ("w_rows", C.c_int64),
        ("num_units", C.c_int32), ("reserved", C.c_int32),
        ("units", C.POINTER(FctpFusedWUnit)), ("status", C.c_void_p),
    ]


class GemmF32x3Args(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B_hi", C.c_void_p), ("B_lo", C.c_void_p), ("bias", C.c_void_p), ("C", C.c_void_p),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("status", C.c_void_p),
    ]


class GemmF32x3TnArgs(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("colsum", C.c_void_p),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
        ("status", C.c_void_p),
    ]


_lib = None


class CueqError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Loads the CUDA library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise CueqError(
            f"{LIB_PATH} is missing: build it with `python -m cuequivariance_b200.build` "
            "(there is no CPU or PyTorch fallback for the CUDA executor)"
        )
    L = C.CDLL(str(LIB_PATH))
    L.cueq_b200_abi_version.restype = C.c_int
    L.cueq_b200_last_error.restype = C.c_char_p
    L.cueq_b200_u1d_plan_create.argtypes = [C.POINTER(U1dDesc), C.POINTER(C.c_void_p)]
    L.cueq_b200_plan_destroy.argtypes = [C.c_void_p]
    L.cueq_b200_plan_destroy.restype = None
    L.cueq_b200_plan_table_bytes.argtypes = [C.c_void_p]
    L.cueq_b200_plan_table_bytes.restype = C.c_size_t
    L.cueq_b200_plan_table_data.argtypes = [C.c_void_p]
    L.cueq_b200_plan_table_data.restype = C.c_void_p
    L.cueq_b200_u1d_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(Buffer), C.c_int32, C.c_void_p]
    L.cueq_b200_segmented_transpose.argtypes = [
        C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
    ]
    L.cueq_b200_cw_num_groups.restype = C.c_int
    L.cueq_b200_cw_group_signature.argtypes = [C.c_int]
    L.cueq_b200_cw_group_signature.restype = C.c_char_p
    L.cueq_b200_cw_group_info.argtypes = [C.c_int] + [C.POINTER(C.c_int32)] * 4
    L.cueq_b200_selftest_fma_peak.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    L.cueq_b200_selftest_fma2_peak.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
    L.cueq_b200_check_index_range.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]
    L.cueq_b200_copy_async.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    L.cueq_b200_enable_peer_access.argtypes = [C.c_int]
    L.cueq_b200_push.argtypes = [C.POINTER(PushArgs), C.c_void_p]
    L.cueq_b200_ipc_export.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]
    L.cueq_b200_ipc_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    L.cueq_b200_ipc_close.argtypes = [C.c_void_p]
    L.cueq_b200_sh_width.argtypes = [C.c_uint32]
    L.cueq_b200_sh_forward.argtypes = [C.POINTER(ShArgs), C.c_void_p]
    L.cueq_b200_sh_backward.argtypes = [C.POINTER(ShArgs), C.c_void_p]
    L.cueq_b200_cw_forward.argtypes = [C.c_int, C.POINTER(CwArgs), C.c_void_p]
    L.cueq_b200_cw_backward.argtypes = [C.c_int, C.POINTER(CwArgs), C.c_void_p]
    L.cueq_b200_cw_forward_noalloc.argtypes = [C.c_int, C.POINTER(CwNoAllocArgs), C.c_void_p]
    L.cueq_b200_u1d_static_find.argtypes = [C.c_char_p]
    L.cueq_b200_u1d_static_find.restype = C.c_int
    L.cueq_b200_u1d_static_name.argtypes = [C.c_int]
    L.cueq_b200_u1d_static_name.restype = C.c_char_p
    L.cueq_b200_u1d_static_launch.argtypes = [C.c_int, C.c_int64, C.c_int32, C.POINTER(Buffer), C.POINTER(C.c_int32),
                                              C.POINTER(C.c_int32), C.c_int32, C.c_void_p]
    L.cueq_b200_gemm_bf16_tn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                         C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]
    L.cueq_b200_gemm_bf16.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
    L.cueq_b200_fctp_build_z.argtypes = [C.POINTER(FctpArgs), C.c_void_p]
    L.cueq_b200_fctp_consume_gz.argtypes = [C.POINTER(FctpArgs), C.c_void_p]
    L.cueq_b200_fctp_fused_forward.argtypes = [C.POINTER(FctpFusedArgs), C.c_void_p]
    L.cueq_b200_fctp_fused_gx.argtypes = [C.POINTER(FctpFusedGxArgs), C.c_void_p]
    L.cueq_b200_fctp_fused_gw.argtypes = [C.POINTER(FctpFusedGwArgs), C.c_void_p]
    L.cueq_b200_gemm_f32x3.argtypes = [C.POINTER(GemmF32x3Args), C.c_void_p]
    L.cueq_b200_gemm_f32x3_tn.argtypes = [C.POINTER(GemmF32x3TnArgs), C.c_void_p]
    L.cueq_b200_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    if L.cueq_b200_abi_version() != 1:
        raise CueqError("libcueq_b200.so has an unexpected ABI version; rebuild it")
    L.cueq_b200_sizeof.restype = C.c_int64
    for which, struct in enumerate((U1dDesc, Buffer, CwArgs, CwNoAllocArgs, GemmArgs, FctpArgs, FctpFusedArgs, FctpFusedTask, FctpFusedGxArgs, FctpFusedUnit, FctpFusedGwArgs, FctpFusedWUnit, GemmF32x3Args, GemmF32x3TnArgs)):
        if L.cueq_b200_sizeof(which) != C.sizeof(struct):
            raise CueqError(f"{struct.__name__}: this binding declares {C.sizeof(struct)} bytes, the library "
                            f"{L.cueq_b200_sizeof(which)}; rebuild the library or update the binding")
    _lib = L
    return L


def check(status: int) -> None:
    if status != 0:
        raise CueqError(lib().cueq_b200_last_error().decode())


_status_words: dict = {}


def status_word(device):
    """One int32 on ``device`` shared by every launch that takes a ``status`` pointer: kernels with
    bounded waits write a non-zero code there instead of hanging (1: a bulk copy of the channelwise
    staging variant ran out of time, 2: a wait inside a tensor-core kernel did).  Launches never read
    it back (that would synchronise); call :func:`check_status` at a point where a sync is acceptable."""
    import torch

    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    t = _status_words.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[dev] = t
    return t


CHECK_INDICES = bool(os.environ.get("CUEQ_B200_CHECK_INDICES"))   # debug mode, see checked_index()


def checked_index(index, rows: int):
    """Debug mode (``CUEQ_B200_CHECK_INDICES=1`` or ``_lib.CHECK_INDICES = True``): a kernel flags every index
    outside ``[0, rows)`` in the device's status word (code 3, reported by :func:`check_status`) and the
    index handed to the product kernels is clamped into range, so that a bad index can neither fault nor
    corrupt memory.  Off by default: index range is the caller's responsibility, as in the reference."""
    if not CHECK_INDICES or index is None or not index.is_cuda or index.numel() == 0:
        return index
    import torch

    with torch.cuda.device(index.device):
        check(lib().cueq_b200_check_index_range(C.c_void_p(index.data_ptr()), index.numel(), int(rows), 1 if index.dtype == torch.int64 else 0,
                                                C.c_void_p(status_word(index.device).data_ptr()),
                                                C.c_void_p(torch.cuda.current_stream(index.device).cuda_stream)))
    return index.clamp(0, max(int(rows) - 1, 0))


def check_status(device=None) -> None:
    """Synchronises and raises :class:`CueqError` if any kernel since the last check reported a wait that
    ran out (its results are then incomplete) or, in index-checking mode, an index out of range.  The word is
    cleared."""
    for dev, t in list(_status_words.items()):
        if device is not None and dev != __import__("torch").device(device):
            continue
        code = int(t.item())
        if code:
            t.zero_()
            if code == 3:
                raise CueqError(f"an index tensor on {dev} pointed outside its buffer (status 3); it was clamped into range, the results are wrong")
            raise CueqError(f"a kernel on {dev} gave up on a bounded wait (status {code}); its outputs are incomplete")


def int32_array(values):
    values = list(values)
    return (C.c_int32 * max(len(values), 1))(*values)


def double_array(values):
    values = list(values)
    return (C.c_double * max(len(values), 1))(*values)
