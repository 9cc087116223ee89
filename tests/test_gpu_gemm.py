"""The hand-written tensor-core GEMM (TMA + tcgen05 + TMEM) against torch on the same bf16
inputs: float32 accumulation of exact bf16 products, so the results agree to float32
rounding of the summation order (rtol 1e-4, atol 1e-3 at K up to 4096)."""
import ctypes as C

import pytest
import torch

from cuequivariance_b200 import _lib

DEV = "cuda:0"

pytestmark = pytest.mark.gpu


def _gemm(a, b, c=None):
    M, K = a.shape
    N = b.shape[0]
    acc = c is not None
    if c is None:
        c = torch.full((M, N), float("nan"), dtype=torch.float32, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    _lib.check(_lib.lib().cueq_b200_gemm_bf16_tn(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, a.stride(0), b.stride(0),
                                                 c.stride(0), 1 if acc else 0, status.data_ptr(),
                                                 C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
    return c


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (128, 64, 256), (300, 128, 512), (1000, 64, 4096), (163840, 64, 4096)])
def test_gemm_bf16_matches_torch(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    got = _gemm(a, b)
    assert torch.allclose(got, ref, rtol=1e-4, atol=1e-3 * (K / 64) ** 0.5), float((got - ref).abs().max())
    # accumulate into an existing C
    got2 = _gemm(a, b, got.clone())
    assert torch.allclose(got2, 2 * ref, rtol=1e-4, atol=2e-3 * (K / 64) ** 0.5)


def _gemm_general(a, b, M, N, K, a_mn=False, b_mn=False, out_bf16=False, rows_per_group=1, group_stride=0, c=None, ldc=None):
    g = _lib.GemmArgs()
    ldc = ldc or N
    if c is None:
        c = torch.zeros((M, N), dtype=torch.bfloat16 if out_bf16 else torch.float32, device=a.device)
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    g.A, g.B, g.C = a.data_ptr(), b.data_ptr(), c.data_ptr()
    g.M, g.N, g.K = M, N, K
    g.lda, g.ldb, g.ldc = a.stride(0), b.stride(0), ldc
    g.rows_per_group, g.group_stride = rows_per_group, group_stride
    g.out_bf16, g.a_mn_major, g.b_mn_major = int(out_bf16), int(a_mn), int(b_mn)
    g.status = status.data_ptr()
    _lib.check(_lib.lib().cueq_b200_gemm_bf16(C.byref(g), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return c


@pytest.mark.parametrize("a_mn,b_mn", [(True, False), (False, True), (True, True)])
def test_gemm_mn_major_operands(a_mn, b_mn):
    M, N, K = 256, 128, 320
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    got = _gemm_general(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, M, N, K, a_mn, b_mn)
    assert torch.allclose(got, ref, rtol=1e-4, atol=3e-3), float((got - ref).abs().max())


def test_gemm_grouped_rows_and_bf16_output():
    M, N, K = 3 * 100, 64, 128
    g = torch.Generator(device="cuda").manual_seed(4)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    # rows (z, k) with k < 3 land at z * 400 + 70 + k * 64 inside a wider row-major buffer
    buf = torch.zeros(100, 400, device="cuda")
    _gemm_general(a, b, M, N, K, rows_per_group=3, group_stride=400, c=buf[:, 8:], ldc=64)
    assert torch.allclose(buf[:, 8 : 8 + 192].reshape(300, 64), ref, rtol=1e-4, atol=2e-3)
    assert torch.count_nonzero(buf[:, :8]) == 0 and torch.count_nonzero(buf[:, 200:]) == 0
    got = _gemm_general(a, b, M, N, K, out_bf16=True)
    assert torch.allclose(got.float(), ref, rtol=2e-2, atol=2e-1)


@pytest.mark.parametrize("M,N,K,bias", [(1000, 2944, 64, True), (300, 132, 32, True), (128, 128, 64, False), (5, 4, 32, True),
                                          (700, 64, 2944, False), (260, 200, 160, True), (64, 36, 96, True)])
def test_linear_f32x3_against_float64(M, N, K, bias):
    """Three-pass TF32 dense layer (csrc/gemm_f32x3.cu) against a float64 matmul of the same float32
    inputs: float32 accuracy, |err| <= 1e-5 of the result's scale (a single TF32 pass is ~1e-3);
    ragged M and N exercise the clipped TMA loads and stores.  Gradients: against torch autograd."""
    from cuequivariance_b200.dense import linear_f32x3, split_tf32

    g = torch.Generator(device=DEV).manual_seed(M + N)
    x = torch.randn(M, K, generator=g, device=DEV, requires_grad=True)
    w = (torch.randn(N, K, generator=g, device=DEV) / 8).requires_grad_(True)
    b = torch.randn(N, generator=g, device=DEV, requires_grad=True) if bias else None
    hi, lo = split_tf32(w.detach())
    assert int((hi.view(torch.int32) & 8191).abs().max()) == 0 and int((lo.view(torch.int32) & 8191).abs().max()) == 0
    assert float((hi + lo - w.detach()).abs().max()) <= 2.0 ** -20 * float(w.detach().abs().max())
    y = linear_f32x3(x, w, b)
    ref = x.detach().double() @ w.detach().double().t() + (b.detach().double() if bias else 0.0)
    scale = float(ref.abs().max())
    assert float((y.detach().double() - ref).abs().max()) <= 1e-5 * scale
    cot = torch.randn(M, N, generator=g, device=DEV)
    got = torch.autograd.grad(y, [x, w] + ([b] if bias else []), cot)
    want = torch.autograd.grad(torch.nn.functional.linear(x, w, b), [x, w] + ([b] if bias else []), cot)
    for a, c in zip(got, want):
        assert float((a - c).abs().max()) <= 1e-4 * max(1.0, float(c.abs().max()))


@pytest.mark.parametrize("K,M,N", [(32, 128, 64), (100, 128, 64), (5000, 2944, 64), (700, 132, 36), (9000, 260, 200)])
def test_gemm_f32x3_tn_against_float64(K, M, N):
    """Row-reduction product a[K, M].T @ b[K, N] with column sums (csrc/gemm_f32x3.cu, the weight / bias
    gradient of a dense layer): float32 accuracy against a float64 product of the same inputs, ragged
    K, M and N included."""
    from cuequivariance_b200.dense import gemm_f32x3_tn

    g = torch.Generator(device=DEV).manual_seed(K + M)
    a = torch.randn(K, M, generator=g, device=DEV)
    b = torch.randn(K, N, generator=g, device=DEV)
    c, cs = gemm_f32x3_tn(a, b, with_colsum=True)
    ref = a.double().t() @ b.double()
    assert float((c.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    ref_cs = a.double().sum(0)
    assert float((cs.double() - ref_cs).abs().max()) <= 1e-5 * max(1.0, float(ref_cs.abs().max()))
    c2 = gemm_f32x3_tn(a[:, : M // 2 // 4 * 4], b)          # a column slice of a wider tensor, no column sums
    assert float((c2.double() - ref[: M // 2 // 4 * 4]).abs().max()) <= 1e-5 * float(ref.abs().max())


def test_bounded_wait_times_out_and_reports():
    """A wait that nothing satisfies must come back by itself: the kernel returns within about a
    second, the shared status word reads 2, `check_status()` raises and clears it, and the device
    keeps working afterwards."""
    import time

    import cuequivariance_b200 as cb
    from cuequivariance_b200._lib import CueqError

    cb.check_status()                                   # clean before
    status = _lib.status_word(DEV)
    cycles = torch.zeros(1, dtype=torch.int64, device=DEV)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _lib.check(_lib.lib().cueq_b200_selftest_bounded_wait(status.data_ptr(), cycles.data_ptr(),
                                                          C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert 0.05 < elapsed < 5.0, elapsed
    assert int(status.item()) == 2 and int(cycles.item()) >= 1 << 30
    with pytest.raises(CueqError):
        cb.check_status()
    cb.check_status()                                   # cleared by the raising call
    a = torch.randn(256, 64, device=DEV)
    from cuequivariance_b200.dense import gemm_f32x3

    y = gemm_f32x3(a, a[:64])
    assert torch.isfinite(y).all()


# ---- CUDA-core kernels around the dense float32 route: coupled operand and its consumer -----------------------
@pytest.mark.parametrize("d1,d2,d3,U,V,pitch_extra,z_dtype", [
    (1, 1, 1, 64, 64, 0, "f32"),       # compile-time kernels, groups of 16 threads per u
    (3, 5, 3, 64, 64, 32, "f32"),      # Z as a column block of a wider matrix
    (5, 5, 5, 24, 32, 0, "f32"),       # fewer u than thread groups
    (7, 3, 5, 40, 128, 0, "f32"),      # a full warp per u
    (3, 3, 1, 17, 16, 4, "f32"),       # four threads per u, odd U
    (5, 7, 7, 8, 16, 0, "f32"),
    (3, 3, 3, 12, 8, 0, "f32"),        # V below 16: generic kernels
    (3, 5, 3, 32, 32, 0, "bf16"),      # bf16 Z: generic kernels
])
def test_fctp_build_and_consume_against_float64(d1, d2, d3, U, V, pitch_extra, z_dtype):
    """Z[(z,k),(u,v)] = sum_ij C[i,j,k] x1[z,i,u] x2[z,j,v]; gx1 / gx2 = its two contractions with gZ
    (the operand kernels of the dense route, csrc/fctp_kernels.cu), float32 against float64 einsum."""
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(d1 * 100 + d2 * 10 + d3 + U + V)
    B = 301
    off1, off2, ld1, ld2 = 5, 3, d1 * U + 9, d2 * V + 4
    x1 = torch.randn(B, ld1, generator=g, device=dev)
    x2 = torch.randn(B, ld2, generator=g, device=dev)
    cg = torch.randn(d1, d2, d3, generator=g, device=dev)
    cg[torch.rand(d1, d2, d3, generator=g, device=dev) < 0.4] = 0.0
    zt = torch.float32 if z_dtype == "f32" else torch.bfloat16
    ldz = U * V + pitch_extra
    Z = torch.full((B * d3, ldz), 7.0, dtype=zt, device=dev)
    cg_host = (C.c_float * (d1 * d2 * d3))(*cg.flatten().tolist())

    def args(zbuf):
        a = _lib.FctpArgs()
        a.x1, a.x2, a.z = x1.data_ptr(), x2.data_ptr(), zbuf.data_ptr()
        a.cg = C.cast(cg_host, C.POINTER(C.c_float))
        a.ld1, a.ld2, a.batch, a.off1, a.off2 = ld1, ld2, B, off1, off2
        a.d1, a.d2, a.d3, a.U, a.V = d1, d2, d3, U, V
        a.x_dtype, a.z_dtype, a.ldz = _lib.F32, (_lib.F32 if z_dtype == "f32" else _lib.BF16), ldz
        return a

    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(_lib.lib().cueq_b200_fctp_build_z(C.byref(args(Z)), st))
    X1 = x1[:, off1 : off1 + d1 * U].double().view(B, d1, U)
    X2 = x2[:, off2 : off2 + d2 * V].double().view(B, d2, V)
    want = torch.einsum("ijk,ziu,zjv->zkuv", cg.double(), X1, X2).reshape(B * d3, U * V)
    tol = 2e-5 if z_dtype == "f32" else 2e-2
    got = Z[:, : U * V].double()
    assert (got - want).abs().max() <= tol * want.abs().max()
    if pitch_extra:
        assert (Z[:, U * V :] == 7.0).all()                      # nothing written beside the block

    gZ = torch.randn(B * d3, ldz, generator=g, device=dev).to(zt)
    gx1 = torch.ones(B, ld1, device=dev)
    gx2 = torch.ones(B, ld2, device=dev)
    a = args(gZ)
    a.gx1, a.gx2 = gx1.data_ptr(), gx2.data_ptr()
    _lib.check(_lib.lib().cueq_b200_fctp_consume_gz(C.byref(a), st))
    G = gZ[:, : U * V].double().view(B, d3, U, V)
    w1 = torch.einsum("ijk,zkuv,zjv->ziu", cg.double(), G, X2).reshape(B, d1 * U)
    w2 = torch.einsum("ijk,zkuv,ziu->zjv", cg.double(), G, X1).reshape(B, d2 * V)
    e1 = (gx1[:, off1 : off1 + d1 * U].double() - 1.0 - w1).abs().max()
    e2 = (gx2[:, off2 : off2 + d2 * V].double() - 1.0 - w2).abs().max()
    assert e1 <= 2e-5 * max(1.0, float(w1.abs().max())), e1
    assert e2 <= 2e-5 * max(1.0, float(w2.abs().max())), e2
    keep1 = torch.ones(ld1, dtype=torch.bool, device=dev)
    keep1[off1 : off1 + d1 * U] = False
    assert (gx1[:, keep1] == 1.0).all() and (gx2[:, : off2] == 1.0).all()   # the neighbouring segments are untouched
