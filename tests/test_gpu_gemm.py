"""tcgen05 GEMM against an fp32 PyTorch product, every operand-major combination."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b):
    return a.float() @ b.float().t()


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(128, 256, 64), (200, 328, 136), (1024, 768, 512)])
def test_gemm_majors(a_mn, b_mn, shape):
    from ringattention_b200.ops import _lib, kernels as K

    M, N, Kd = shape
    torch.manual_seed(0)
    a = torch.randn(M, Kd, device="cuda").bfloat16()
    b = torch.randn(N, Kd, device="cuda").bfloat16()
    A = a.t().contiguous() if a_mn else a
    B = b.t().contiguous() if b_mn else b
    c = K.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = _ref(a, b)
    assert (c.float() - ref).abs().max() <= 0.01 * ref.abs().max() + 1e-3


def test_gemm_residual_and_fp32_accumulate():
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(1)
    a = torch.randn(256, 320, device="cuda").bfloat16()
    b = torch.randn(512, 320, device="cuda").bfloat16()
    r = torch.randn(256, 512, device="cuda").bfloat16()
    c = K.gemm(a, b, residual=r)
    ref = _ref(a, b) + r.float()
    assert (c.float() - ref).abs().max() <= 0.01 * ref.abs().max()
    acc = torch.randn(256, 512, device="cuda")
    acc0 = acc.clone()
    K.gemm(a, b, out=acc, residual=acc)
    assert torch.allclose(acc, acc0 + _ref(a, b), atol=2e-3, rtol=1e-4)


def test_linear_fwd_dgrad_wgrad_match_autograd():
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(2)
    x = torch.randn(384, 256, device="cuda").bfloat16()
    w = torch.randn(512, 256, device="cuda").bfloat16()
    dy = torch.randn(384, 512, device="cuda").bfloat16()
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    (xf @ wf.t()).backward(dy.float())
    y = K.linear_fwd(x, w)
    dx = K.linear_dgrad(dy, w)
    dw = torch.zeros(512, 256, device="cuda")
    K.linear_wgrad(dy, x, dw)
    assert (y.float() - (xf @ wf.t())).abs().max() <= 0.01 * (xf @ wf.t()).abs().max()
    assert (dx.float() - xf.grad).abs().max() <= 0.01 * xf.grad.abs().max()
    assert torch.allclose(dw, wf.grad, atol=2e-2, rtol=1e-3)
