"""tcgen05 GEMM against a PyTorch fp32 reference, all four operand layouts, ragged tails, split-K."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A @ B


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 64, 256), (256, 512, 256, 256), (200, 328, 136, 128),
                                      (1000, 1536, 1536, 0), (64, 72, 8, 64), (4096, 2048, 1536, 256)])
def test_gemm_layouts(a_mn, b_mn, M, N, K, bn):
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops.gemm import gemm

    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("leading dimension must be a multiple of 8")
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    _lib.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_gemm_bias_residual():
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops.gemm import gemm

    torch.manual_seed(1)
    M, N, K = 384, 640, 320
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm(a, b, bias=bias, residual=res)
    _lib.check_status()
    ref = a.float() @ b.float().t() + bias.float() + res.float()
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2


def test_gemm_f32_accumulate_splitk():
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops.gemm import gemm

    torch.manual_seed(2)
    T, N, K = 2048, 256, 384
    dy = torch.randn(T, N, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
    grad = torch.ones(N, K, device="cuda", dtype=torch.float32)
    gemm(dy, x, a_mn=True, b_mn=True, out=grad, accumulate=True, k_splits=4)
    _lib.check_status()
    ref = 1.0 + dy.float().t() @ x.float()
    assert (grad - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3


@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (300, 1536, 1024), (4096, 2048, 1536), (64, 72, 144)])
def test_gemm_e4m3_matches_dequantised_reference(M, N, K):
    """fp8 tcgen05 GEMM against an fp32 matmul of the de-quantised operands (same rounding of the inputs, so only
    the accumulation order and the bf16 output rounding differ)."""
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops.fp8 import Fp8Linear, gemm_e4m3, quantize_e4m3
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    aq, sa = quantize_e4m3(a)
    bq, sb = quantize_e4m3(b)
    assert abs(float(sa) - float(a.float().abs().max()) / 448) < 1e-6
    # quantisation itself: matches torch's e4m3 cast of the scaled tensor
    ref_q = (a.float() / sa).to(torch.float8_e4m3fn)
    assert (aq.float() - ref_q.float()).abs().max().item() <= 1e-6 * 448 + (ref_q.float().abs().max().item() * 0.07)
    out = gemm_e4m3(aq, sa, bq, sb, bias=bias)
    _lib.check_status()
    ref = (aq.float() * sa) @ (bq.float() * sb).t() + bias.float()
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err
    # end to end against the bf16 product: fp8 rounding error only
    y = Fp8Linear(b, bias)(a)
    full = a.float() @ b.float().t() + bias.float()
    rel = ((y.float() - full).norm() / full.norm()).item()
    assert rel < 6e-2, rel
