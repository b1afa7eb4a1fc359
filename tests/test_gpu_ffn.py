"""Kernel-backed blockwise feed-forward: the GEMM with the SwiGLU epilogue, the chunk loop with recomputation
and the public ``blockwise_feedforward`` against the un-chunked PyTorch feed-forward, gradients included."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,F,Kd", [(300, 512, 256), (1024, 1376, 512), (128, 200, 64)])
def test_gemm_swiglu_epilogue_matches_two_pass(M, F, Kd):
    from ringattention_b200.ops import _lib, kernels as K

    torch.manual_seed(0)
    x = torch.randn(M, Kd, device="cuda").bfloat16()
    w = (torch.randn(2 * F, Kd, device="cuda") * 0.05).bfloat16()
    fused = K.linear_swiglu(x, w)
    two_pass = K.swiglu_fwd(K.linear_fwd(x, w))
    torch.cuda.synchronize()
    _lib.check_status()
    # both round gate and up to bf16 before the activation: identical up to the order of the k-loop (none here)
    assert torch.equal(fused, two_pass)
    gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    assert (fused.float() - ref).abs().max() <= 0.02 * ref.abs().max() + 1e-3


@pytest.mark.parametrize("policy,pre_remat", [("nothing_saveable", True), ("nothing_saveable", False),
                                              ("everything_saveable", False)])
def test_blockwise_feedforward_on_the_kernels(policy, pre_remat):
    """ringattention_jax.py:333-352 with a FusedSwiGLU module: same output and gradients as the un-chunked
    PyTorch feed-forward."""
    import ringattention_b200 as rab
    from ringattention_b200.ops import _lib
    from ringattention_b200.ops.ffn import FusedSwiGLU

    torch.manual_seed(1)
    B, S, d, F = 2, 512, 256, 640
    ff = FusedSwiGLU(d, F, seed=3)
    x = torch.randn(B, S, d, device="cuda").bfloat16().requires_grad_(True)
    dy = torch.randn(B, S, d, device="cuda").bfloat16()
    y = rab.blockwise_feedforward(ff, x, 128, policy=policy, pre_remat=pre_remat)
    y.backward(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    xr = x.detach().float().requires_grad_(True)
    wg = ff.weight_gate_up.detach().float().requires_grad_(True)
    wd = ff.weight_down.detach().float().requires_grad_(True)
    gu = xr @ wg.t()
    yr = (torch.nn.functional.silu(gu[..., :F]) * gu[..., F:]) @ wd.t()
    yr.backward(dy.float())
    rel = lambda a, b: ((a.float() - b).abs().max() / (b.abs().max() + 1e-9)).item()
    assert rel(y, yr) < 0.02
    assert rel(x.grad, xr.grad) < 0.02
    assert rel(ff.weight_gate_up.grad, wg.grad) < 0.02
    assert rel(ff.weight_down.grad, wd.grad) < 0.02
    # un-chunked call of the module: same function
    assert rel(ff(x.detach()), yr) < 0.02


def test_blockwise_feedforward_still_takes_any_callable():
    import ringattention_b200 as rab

    lin = torch.nn.Linear(64, 64).cuda()
    x = torch.randn(2, 256, 64, device="cuda")
    y = rab.blockwise_feedforward(lambda t: torch.tanh(lin(t)), x, 64)
    assert torch.allclose(y, torch.tanh(lin(x)), atol=1e-5)
