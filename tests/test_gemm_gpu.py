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


@pytest.mark.parametrize("M,I,K,bn", [(128, 8960, 1536, 128), (1000, 512, 256, 0), (4096, 1024, 1536, 256),
                                      (37, 128, 72, 128), (10240, 8960, 1536, 0), (2500, 2048, 264, 256), (2700, 1920, 512, 0)])
def test_gemm_swiglu_epilogue(M, I, K, bn):
    """SwiGLU fused into the GEMM epilogue (two B boxes per stage) against fp32 PyTorch; the optional gate / up output
    and the autograd wrapper against the unfused composition."""
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.ops import functional as F
    from openrlhf_b200.ops.gemm import gemm_swiglu

    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda") / K ** 0.5).bfloat16()
    y, gu = gemm_swiglu(x, w, want_gate_up=True, bn=bn)
    _lib.check_status()
    ref_gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(ref_gu[:, :I]) * ref_gu[:, I:]
    assert (gu.float() - ref_gu).abs().max().item() < 0.02 * ref_gu.abs().max().item()
    assert (y.float() - ref).abs().max().item() < 0.02 * ref.abs().max().item()
    y2, none = gemm_swiglu(x, w, bn=bn)
    assert none is None and torch.equal(y, y2)
    if M > 2000:
        return
    # autograd: same gradients as linear followed by the separate SwiGLU kernel
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xb, wb = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    dy = torch.randn(M, I, device="cuda", dtype=torch.bfloat16)
    F.linear_swiglu(xa, wa).backward(dy)
    F.swiglu(F.linear(xb, wb)).backward(dy)
    _lib.check_status()
    assert (xa.grad.float() - xb.grad.float()).abs().max().item() <= 0.02 * xb.grad.float().abs().max().item()
    assert (wa.grad.float() - wb.grad.float()).abs().max().item() <= 0.02 * wb.grad.float().abs().max().item()


def _gemm2(a, b, *, a_mn=False, b_mn=False, bias=None, residual=None, out=None, accumulate=False, k_splits=1, bn=256):
    """The CTA-pair kernel through its C symbol (ops.gemm only routes large shapes to it)."""
    import ctypes

    from openrlhf_b200.ops import _lib

    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=torch.bfloat16)
    f32 = out.dtype == torch.float32
    rc = _lib.lib().b200_gemm2_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(residual), ctypes.c_int(M), ctypes.c_int(N),
        ctypes.c_int(K), ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(out.stride(0)),
        ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)), ctypes.c_int(int(f32)), ctypes.c_int(int(accumulate)),
        ctypes.c_int(k_splits), ctypes.c_float(1.0), ctypes.c_int(bn), _lib.ptr(_lib.status_word(a.device)),
        _lib.stream_ptr())
    assert rc == 0, rc
    return out


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K,bn", [(256, 256, 64, 256), (512, 768, 256, 256), (1000, 1536, 1544, 256),
                                      (2048, 1024, 512, 128), (4096, 2304, 1536, 256), (136, 264, 72, 128)])
def test_gemm_cta_pair_layouts(a_mn, b_mn, M, N, K, bn):
    """tcgen05.mma.cta_group::2 kernel (two CTAs per 256-row tile) against fp32 PyTorch: all operand layouts, ragged
    M / N / K tails (the odd CTA of the last pair may hold no valid row at all), one and many tiles per pair."""
    from openrlhf_b200.ops import _lib

    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    out = _gemm2(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_gemm_cta_pair_epilogues():
    from openrlhf_b200.ops import _lib

    torch.manual_seed(3)
    M, N, K = 768, 640, 320
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    out = _gemm2(a, b, bias=bias, residual=res)
    ref = a.float() @ b.float().t() + bias.float() + res.float()
    assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    # weight-gradient form: fp32 accumulation into an existing buffer, split along the token dimension
    T, Nw, Kw = 4096, 512, 384
    dy = torch.randn(T, Nw, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, Kw, device="cuda", dtype=torch.bfloat16)
    grad = torch.ones(Nw, Kw, device="cuda", dtype=torch.float32)
    _gemm2(dy, x, a_mn=True, b_mn=True, out=grad, accumulate=True, k_splits=4)
    torch.cuda.synchronize()
    _lib.check_status()
    want = 1.0 + dy.float().t() @ x.float()
    assert (grad - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-2
