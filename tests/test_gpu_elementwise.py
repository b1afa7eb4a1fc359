"""Driver kernels (norm, rope, swiglu, embedding, loss, optimizer, casts) against fp32 PyTorch."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def test_rmsnorm_fwd_bwd():
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(0)
    for rows, d in ((300, 512), (257, 4096), (64, 1024)):
        x = torch.randn(rows, d, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
        dy = torch.randn(rows, d, device="cuda").bfloat16()
        dres = torch.randn(rows, d, device="cuda").bfloat16()
        xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
        yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
        yr.backward(dy.float())
        y, rstd = K.rmsnorm_fwd(x, w, 1e-6)
        assert (y.float() - yr).abs().max() < 0.05
        dw = torch.zeros(d, device="cuda")
        dx = K.rmsnorm_bwd(dy, x, w, rstd, dw, dres=dres)
        assert (dx.float() - (xf.grad + dres.float())).abs().max() < 0.06
        assert (dw - wf.grad).abs().max() <= 0.02 * wf.grad.abs().max() + 0.05


def test_rope_roundtrip_and_reference():
    from llama_torch import rope_torch
    from ringattention_b200.ops import kernels as K
    from ringattention_b200.ops.flash import Positions

    torch.manual_seed(1)
    B, S, H, D = 2, 256, 6, 128
    buf = torch.randn(B, S, 3 * H, D, device="cuda").bfloat16()
    x = buf[:, :, :2 * H]  # strided view, like q|k inside a fused qkv buffer
    x0 = x.clone()
    pos = Positions(1000, 5000, 128)  # two runs, as in the zig-zag layout
    ref = rope_torch(x0, pos.tensor(S, "cuda"), 10000.0)
    K.rope_(x, pos, 10000.0)
    assert (x.float() - ref.float()).abs().max() < 0.04
    assert torch.equal(buf[:, :, 2 * H:], buf[:, :, 2 * H:])  # v part untouched by construction
    K.rope_(x, pos, 10000.0, inverse=True)
    assert (x.float() - x0.float()).abs().max() < 0.05


def test_swiglu_fwd_bwd():
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(2)
    rows, Fd = 200, 1536
    gu = torch.randn(rows, 2 * Fd, device="cuda").bfloat16()
    dh = torch.randn(rows, Fd, device="cuda").bfloat16()
    guf = gu.float().requires_grad_(True)
    h_ref = F.silu(guf[:, :Fd]) * guf[:, Fd:]
    h_ref.backward(dh.float())
    h = K.swiglu_fwd(gu)
    assert (h.float() - h_ref).abs().max() < 0.05
    d = K.swiglu_bwd_(gu.clone(), dh)
    assert (d.float() - guf.grad).abs().max() < 0.06


def test_embedding_and_xent():
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(3)
    V, d, n = 1024, 256, 500
    table = torch.randn(V, d, device="cuda").bfloat16()
    tok = torch.randint(0, V, (n,), device="cuda", dtype=torch.int32)
    out = K.embedding_fwd(tok, table)
    assert torch.equal(out, table[tok.long()])
    dy = torch.randn(n, d, device="cuda").bfloat16()
    dt = torch.zeros(V, d, device="cuda")
    K.embedding_bwd(tok, dy, dt)
    ref = torch.zeros(V, d, device="cuda").index_add_(0, tok.long(), dy.float())
    assert torch.allclose(dt, ref, atol=1e-3)
    logits = (torch.randn(n, V, device="cuda") * 3).bfloat16()
    tgt = torch.randint(0, V, (n,), device="cuda", dtype=torch.int32)
    tgt[::7] = -1
    lf = logits.float().requires_grad_(True)
    valid = tgt >= 0
    lref = F.cross_entropy(lf[valid], tgt[valid].long(), reduction="none")
    (lref.sum() * 0.5).backward()
    work = logits.clone()
    loss = K.xent_fwd_bwd_(work, tgt, 0.5)
    assert torch.allclose(loss[valid], lref, atol=2e-2)
    assert bool((loss[~valid] == 0).all())
    assert (work.float() - lf.grad).abs().max() < 5e-3


def test_adamw_matches_torch():
    from ringattention_b200.ops import kernels as K

    torch.manual_seed(4)
    n = 4096
    p = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref_p.grad = g.clone()
        opt.step()
        K.adamw_(p, m, v, g, p16, step=step, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                 weight_decay=0.1, decay_end=n)
    assert torch.allclose(p, ref_p.detach(), atol=1e-5)
    assert torch.allclose(p16.float(), p, atol=2e-2)
    # clipping driven by a device-side squared norm
    g = torch.randn(n, device="cuda") * 10
    s = torch.zeros(1, device="cuda")
    K.sumsq(g, s)
    assert abs(s.item() - g.pow(2).sum().item()) / g.pow(2).sum().item() < 1e-4


def test_casts():
    from ringattention_b200.ops import kernels as K

    src = torch.randn(64, 256, device="cuda")
    big = torch.zeros(64, 3, 256, device="cuda", dtype=torch.bfloat16)
    K.cast_f32_to_bf16(src, big[:, 1])
    assert torch.equal(big[:, 1], src.bfloat16()) and bool((big[:, 0] == 0).all())
    back = torch.empty(64 * 256, device="cuda")
    K.cast_bf16_to_f32(big[:, 1].contiguous().view(-1), back)
    assert torch.equal(back.view(64, 256), src.bfloat16().float())
