"""tcgen05 GEMM numerics against a plain fp32 matmul (GPU only)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,N,K", [(128, 128, 64), (128, 128, 256), (256, 384, 2560), (200, 324, 2560), (4096, 512, 2560),
                                   (77, 130, 328)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tc_matches_fp32(T, N, K, out_dtype):
    from qwb200.ops import kernels as K_
    g = torch.Generator(device="cuda").manual_seed(T + N + K)
    A = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    ldc = (N + 7) // 8 * 8 + 8
    out = torch.full((T, ldc), 768.0, dtype=out_dtype, device="cuda")      # guard columns detect stray writes
    K_.gemm_bf16_tc(A, W, out=out[:, :N])
    torch.cuda.synchronize()
    ref = A.float() @ W.float().T
    assert torch.all(out[:, N:].float() == 768.0)
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    err = float((out[:, :N].float() - ref).abs().max() / ref.abs().max())
    assert err < tol, err
