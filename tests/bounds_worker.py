"""Run under RINGATTN_B200_BOUNDS_CHECK=1 by test_gpu_bounds.py: every kernel family at ragged shapes, outputs
inside canary-padded buffers; prints one line ``BOUNDS {...}`` with what was found."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ringattention_b200.ops import _lib, flash, kernels as K  # noqa: E402

GUARD = 512
_checks = []


def canary(shape, dtype, fill=None):
    """A tensor of ``shape`` carved out of a larger buffer whose 512 elements on either side hold a sentinel."""
    n = 1
    for s in shape:
        n *= s
    sentinel = 12345 if dtype in (torch.int32,) else 7.25
    buf = torch.full((n + 2 * GUARD,), sentinel, device="cuda", dtype=dtype)
    view = buf[GUARD:GUARD + n].view(shape)
    if fill is not None:
        view.copy_(fill)
    _checks.append((buf, n, sentinel))
    return view


def canaries_intact():
    bad = 0
    for buf, n, sentinel in _checks:
        bad += int((buf[:GUARD] != sentinel).sum()) + int((buf[GUARD + n:] != sentinel).sum())
    return bad == 0


def main():
    torch.manual_seed(0)
    dev = "cuda"
    bf = torch.bfloat16
    # ---- GEMM family at sizes that are multiples of nothing in particular
    M, N, Kd = 300, 200, 136
    a, b = torch.randn(M, Kd, device=dev).to(bf), torch.randn(N, Kd, device=dev).to(bf)
    c = K.gemm(a, b, out=canary((M, N), bf))
    assert (c.float() - a.float() @ b.float().t()).abs().max() < 0.5
    K.gemm(a, b, out=canary((M, N), torch.float32))
    a2, b2 = torch.randn(Kd, 304, device=dev).to(bf), torch.randn(Kd, 208, device=dev).to(bf)  # (K, M), (K, N)
    K.gemm(a2, b2, a_mn=True, b_mn=True, out=canary((304, 208), bf))
    w = (torch.randn(2 * 200, Kd, device=dev) * 0.1).to(bf)
    K.linear_swiglu(a, w, out=canary((M, 200), bf))
    # ---- attention forward / backward, ragged, with offsets, segments and a boolean mask
    for D, Sq, Sk in ((128, 300, 777), (64, 129, 255)):
        B, H = 2, 3
        q = torch.randn(B, Sq, H, D, device=dev).to(bf)
        k, v = torch.randn(B, Sk, H, D, device=dev).to(bf), torch.randn(B, Sk, H, D, device=dev).to(bf)
        do = torch.randn(B, Sq, H, D, device=dev).to(bf)
        seg_all = torch.cumsum((torch.rand(B, Sk, device=dev) < 0.01).int(), 1).int()
        ms = flash.MaskSpec(causal_block_size=1, q_pos=flash.Positions(Sk - Sq), k_pos=flash.Positions(0),
                            seg_q=seg_all[:, Sk - Sq:].contiguous(), seg_k=seg_all.contiguous())
        ms.seg_q_mm, ms.seg_k_mm = flash.seg_tile_minmax(ms.seg_q), flash.seg_tile_minmax(ms.seg_k)
        keep = torch.rand(B, 1, Sq, Sk, device=dev) < 0.9
        ms.keep_q, ms.keep_k = flash.pack_mask(keep)
        out, lse = flash.flash_fwd(q, k, v, ms, out=canary((B, Sq, H, D), bf), lse_out=canary((B, H, Sq), torch.float32))
        lse2, delta = flash.flash_bwd_prep(out, do, lse)
        dq_acc = canary((B, Sq, H, D), torch.float32, fill=0.0)
        flash.flash_bwd(q, k, v, do, lse2, delta, ms, dq_acc, canary((B, Sk, H, D), bf), canary((B, Sk, H, D), bf))
    # ---- memory-bound kernels
    rows, d = 37, 512
    x = torch.randn(rows, d, device=dev).to(bf)
    g = torch.ones(d, device=dev).to(bf)
    y, rstd = K.rmsnorm_fwd(x, g, 1e-6, out=canary((rows, d), bf), rstd=canary((rows,), torch.float32))
    K.rmsnorm_bwd(x, x, g, rstd, canary((d,), torch.float32, fill=0.0), out=canary((rows, d), bf))
    xr = canary((1, 37, 4, 64), bf, fill=torch.randn(1, 37, 4, 64, device=dev).to(bf))
    K.rope_(xr, flash.Positions(5, 900, 16), 10000.0)
    gu = torch.randn(rows, 2 * 264, device=dev).to(bf)
    K.swiglu_fwd(gu, out=canary((rows, 264), bf))
    K.swiglu_bwd_(canary((rows, 2 * 264), bf, fill=gu), torch.randn(rows, 264, device=dev).to(bf))
    table = torch.randn(1000, 64, device=dev).to(bf)
    tok = torch.randint(0, 1000, (77,), device=dev, dtype=torch.int32)
    K.embedding_fwd(tok, table, out=canary((77, 64), bf))
    K.embedding_bwd(tok, torch.randn(77, 64, device=dev).to(bf), canary((1000, 64), torch.float32, fill=0.0))
    logits = canary((33, 1000), bf, fill=torch.randn(33, 1000, device=dev).to(bf))
    tgt = torch.randint(-1, 1000, (33,), device=dev, dtype=torch.int32)
    K.xent_fwd_bwd_(logits, tgt, 0.5, loss=canary((33,), torch.float32))
    n = 4100
    p32, m, vv, gr = [canary((n,), torch.float32, fill=torch.randn(n, device=dev)) for _ in range(4)]
    vv.abs_()
    K.adamw_(p32, m, vv, gr, canary((n,), bf), step=1, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
             decay_end=4000)
    K.cast_f32_to_bf16(torch.randn(19, 72, device=dev), canary((19, 72), bf))
    # ---- decode family: split-KV attention over a heads-major cache, merge, weight-streaming linears with their
    # prologues, RoPE + cache append
    from ringattention_b200.ops import decode as Dk

    B, H, D, S = 2, 3, 128, 777
    cache = canary((B, 2, H, S, D), bf, fill=torch.randn(B, 2, H, S, D, device=dev).to(bf))
    ck, cv = cache[:, 0].permute(0, 2, 1, 3), cache[:, 1].permute(0, 2, 1, 3)
    qd = torch.randn(B, 1, H, D, device=dev).to(bf)
    o_part, lse_part = Dk.decode_partial(qd, ck, cv, q_pos0=S, k_pos0=0)
    Dk.merge_partials(o_part, lse_part, H, 1, out=canary((B, 1, H, D), bf))
    xs_, ws_ = torch.randn(3, 520, device=dev).to(bf), (torch.randn(203, 520, device=dev) * 0.05).to(bf)
    K.small_m_linear(xs_, ws_, out=canary((3, 203), bf))
    K.norm_linear(xs_, torch.ones(520, device=dev).to(bf), 1e-6, ws_, out=canary((3, 203), bf))
    K.swiglu_linear(torch.randn(3, 1040, device=dev).to(bf), ws_, out=canary((3, 203), bf))
    qkv = canary((B, 1, 3, H, D), bf, fill=torch.randn(B, 1, 3, H, D, device=dev).to(bf))
    K.rope_append(qkv, ck, cv, torch.tensor([S - 1, 0], device=dev, dtype=torch.int64), 10000.0)
    K.rope_append(qkv, ck, cv, torch.tensor([S + 5, 0], device=dev, dtype=torch.int64), 10000.0)  # not on this shard
    torch.cuda.synchronize()
    _lib.check_status()
    clean = _lib.bounds_report(reset=True)
    # ---- the mechanism itself: a token id outside the vocabulary is clamped by the kernel (no bad access ever
    # happens) and, in the checked build, recorded
    bad_tok = tok.clone()
    bad_tok[3] = 5000
    K.embedding_fwd(bad_tok, table, out=canary((77, 64), bf))
    seeded = _lib.bounds_report(reset=True)
    print("BOUNDS " + json.dumps({"clean": clean, "seeded": seeded, "canaries_intact": canaries_intact()}), flush=True)


if __name__ == "__main__":
    main()
