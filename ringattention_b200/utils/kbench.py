"""Kernel micro-benchmarks with CUDA-event timing and roofline fractions.

    python -m ringattention_b200.utils.kbench --kernel attn_fwd --seq 32768 --heads 32
    python -m ringattention_b200.utils.kbench --kernel attn_bwd --seq 16384 --heads 16 --iters 1 --warmup 1
    python -m ringattention_b200.utils.kbench --kernel gemm --m 65536 --n 4096 --k 4096

Timing: ``--warmup`` untimed launches (>= 3 by default), then ``--iters`` launches between two CUDA
events on the launching stream with a synchronize on both sides. The operands of the attention
cases are far larger than the 126 MB L2 at the default sizes; ``--flush-l2`` writes a 256 MB buffer
between iterations (then every iteration is timed on its own and the mean is reported).
The denominators come from ``MEASURED_PEAKS.json`` at the repository root when present (fractions
"of measured"), else 1590 TFLOP/s and 6650 GB/s ("of fallback").
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import _lib, flash
from ..ops import kernels as K

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0, "fallback"


def time_launches(fn, warmup: int, iters: int, flush_l2: bool) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if not flush_l2:
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters
    junk = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    total = 0.0
    for _ in range(iters):
        junk.fill_(1)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--kernel", required=True, choices=["attn_fwd", "attn_bwd", "gemm", "gemm_dgrad", "gemm_wgrad", "decode", "small_m_linear", "sdpa_fwd", "sdpa_bwd"])
    ap.add_argument("--seq", type=int, default=32768)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--causal", type=int, default=1)
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--mean-doc-len", type=int, default=0,
                    help="attention kernels: packed documents with geometric lengths of this mean (segment ids); "
                         "-1 = segment ids present but all equal")
    args = ap.parse_args(argv)
    peak_tf, peak_gbs, how = peaks()
    torch.manual_seed(0)
    dev = "cuda"
    res = {"kernel": args.kernel, "denominator": how}
    if args.kernel.startswith("attn"):
        B, S, H, D = args.batch, args.seq, args.heads, args.head_dim
        q = torch.randn(B, S, H, D, device=dev).bfloat16()
        k, v, do = torch.randn_like(q), torch.randn_like(q), torch.randn_like(q)
        ms = flash.MaskSpec(causal_block_size=args.causal, q_pos=flash.Positions(0), k_pos=flash.Positions(0))
        out = torch.empty_like(q)
        lse = torch.empty(B, H, S, device=dev)
        frac = 0.5 if args.causal else 1.0
        if args.mean_doc_len:
            from ..trainer import geometric_segment_ids

            if args.mean_doc_len > 0:
                seg = geometric_segment_ids(B, S, args.mean_doc_len, torch.Generator().manual_seed(0)).to(dev)
            else:
                seg = torch.zeros(B, S, dtype=torch.int32, device=dev)
            ms.seg_q = ms.seg_k = seg
            ms.seg_q_mm = ms.seg_k_mm = flash.seg_tile_minmax(seg)
            # visible (q, k) pairs: same document and (if causal) k <= q
            ln = torch.bincount(seg.flatten().long() + (torch.arange(B, device=dev)[:, None] * (int(seg.max()) + 1)).expand(B, S).flatten()).double()
            pairs = float(((ln * (ln + 1) / 2) if args.causal else ln * ln).sum())
            frac = pairs / (float(B) * S * S)
            res["visible_fraction"] = round(frac, 5)
        if args.kernel == "attn_fwd":
            fn = lambda: flash.flash_fwd(q, k, v, ms, out=out, lse_out=lse)
            flops = 4.0 * B * S * S * H * D * frac
            bytes_ = 4.0 * q.numel() * 2
        else:
            flash.flash_fwd(q, k, v, ms, out=out, lse_out=lse)
            lse2, delta = flash.flash_bwd_prep(out, do, lse)
            dq_acc = torch.zeros(B, S, H, D, device=dev)
            dk, dv = torch.empty_like(q), torch.empty_like(q)
            fn = lambda: flash.flash_bwd(q, k, v, do, lse2, delta, ms, dq_acc, dk, dv)
            flops = 10.0 * B * S * S * H * D * frac
            bytes_ = 6.0 * q.numel() * 2 + q.numel() * 4
        res.update(shape=[B, S, H, D], causal=args.causal)
    elif args.kernel.startswith("sdpa"):
        # library comparison: torch.nn.functional.scaled_dot_product_attention (cuDNN / flash backend chosen
        # by torch) on the same shape; not used by the framework
        import torch.nn.functional as F

        B, S, H, D = args.batch, args.seq, args.heads, args.head_dim
        q, k, v = [torch.randn(B, S, H, D, device=dev).bfloat16().transpose(1, 2).requires_grad_(True) for _ in range(3)]
        frac = 0.5 if args.causal else 1.0
        if args.kernel == "sdpa_fwd":
            def fn():
                with torch.no_grad():
                    F.scaled_dot_product_attention(q, k, v, is_causal=bool(args.causal))
            flops = 4.0 * B * S * S * H * D * frac
        else:
            o = F.scaled_dot_product_attention(q, k, v, is_causal=bool(args.causal))
            do = torch.randn_like(o)
            fn = lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
            flops = 10.0 * B * S * S * H * D * frac
        bytes_ = 4.0 * q.numel() * 2
        res.update(shape=[B, S, H, D], causal=args.causal, library=True)
    elif args.kernel == "decode":
        # split-KV decode attention over one cache shard: --seq cache rows, one query row per sequence
        from ..ops import decode as Dk

        B, S, H, D = args.batch, args.seq, args.heads, args.head_dim
        cache = torch.randn(B, S, 2, H, D, device=dev).bfloat16()
        q = torch.randn(B, 1, H, D, device=dev).bfloat16()
        fn = lambda: Dk.decode_partial(q, cache[:, :, 0], cache[:, :, 1], q_pos0=S, k_pos0=0)
        flops = 4.0 * B * S * H * D
        bytes_ = 2.0 * B * S * H * D * 2
        res.update(shape=[B, S, H, D], splits=Dk.default_splits(S, B, H))
    elif args.kernel == "small_m_linear":
        # y[M, N] = x[M, K] W[N, K]^T with M <= 8 (decode-time projections): weight bandwidth is the roofline
        M, N, Kd = min(args.m, 8), args.n, args.k
        ws = [torch.randn(N, Kd, device=dev).bfloat16() for _ in range(8)]  # rotate so that L2 does not help
        x = torch.randn(M, Kd, device=dev).bfloat16()
        turn = [0]

        def fn():
            turn[0] = (turn[0] + 1) % len(ws)
            K.small_m_linear(x, ws[turn[0]])

        flops = 2.0 * M * N * Kd
        bytes_ = 2.0 * N * Kd
        res.update(shape=[M, N, Kd])
    else:
        M, N, Kd = args.m, args.n, args.k
        if args.kernel == "gemm":
            a = torch.randn(M, Kd, device=dev).bfloat16()
            b = torch.randn(N, Kd, device=dev).bfloat16()
            c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: K.gemm(a, b, out=c)
        elif args.kernel == "gemm_dgrad":  # dx[M,N] = dy[M,K] W[K,N]
            a = torch.randn(M, Kd, device=dev).bfloat16()
            b = torch.randn(Kd, N, device=dev).bfloat16()
            c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: K.gemm(a, b, b_mn=True, out=c)
        else:  # dW[M,N] += dy[K,M]^T x[K,N], fp32 accumulate
            a = torch.randn(Kd, M, device=dev).bfloat16()
            b = torch.randn(Kd, N, device=dev).bfloat16()
            c = torch.zeros(M, N, device=dev, dtype=torch.float32)
            fn = lambda: K.gemm(a, b, a_mn=True, b_mn=True, out=c, residual=c)
        flops = 2.0 * M * N * Kd
        bytes_ = 2.0 * (M * Kd + N * Kd) + c.element_size() * M * N
        res.update(shape=[M, N, Kd])
    ms_t = time_launches(fn, args.warmup, args.iters, args.flush_l2)
    _lib.check_status()
    tf = flops / ms_t / 1e9
    res.update(ms=round(ms_t, 4), tflops=round(tf, 1), frac_of_bf16_peak=round(tf / peak_tf, 3),
               algorithmic_gb=round(bytes_ / 1e9, 3), gbs=round(bytes_ / ms_t / 1e6, 1),
               frac_of_hbm_peak=round(bytes_ / ms_t / 1e6 / peak_gbs, 3), iters=args.iters,
               warmup=args.warmup, flush_l2=args.flush_l2)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
