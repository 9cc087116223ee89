"""The hand-written tensor-core GEMM (TMA + tcgen05 + TMEM) against torch on the same bf16
inputs: float32 accumulation of exact bf16 products, so the results agree to float32
rounding of the summation order (rtol 1e-4, atol 1e-3 at K up to 4096)."""
import ctypes as C

import pytest
import torch

from cuequivariance_b200 import _lib

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
