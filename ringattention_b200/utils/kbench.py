"""Kernel micro-benchmarks with CUDA-event timing and roofline fractions.

    python -m ringattention_b200.utils.kbench --kernel attn_fwd --seq 32768 --heads 32
    python -m ringattention_b200.utils.kbench --kernel attn_bwd --seq 16384 --heads 16 --iters 1 --warmup 1
    python -m ringattention_b200.utils.kbench --kernel gemm --m 65536 --n 4096 --k 4096
    python -m ringattention_b200.utils.kbench --kernel memory_bound --m 65536     # every memory-bound kernel, 7B shapes

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


def memory_bound_table(args, peak_gbs: float, how: str) -> int:
    """CUDA-event GB/s of every memory-bound kernel of the driver at the 7B shapes (``--m`` token rows, d_model
    4096, d_ff 11008, vocab 32000): one JSON line per kernel with its algorithmic bytes (each operand read or
    written once) and the fraction of the copy bandwidth. The operands exceed the 126 MB L2 at the default size."""
    dev = "cuda"
    M, d, F, V, H, D = args.m, 4096, 11008, 32000, 32, 128
    bf = torch.bfloat16
    x = torch.randn(M, d, device=dev).to(bf)
    g = torch.ones(d, device=dev).to(bf)
    y, rstd = K.rmsnorm_fwd(x, g, 1e-6)
    dw = torch.zeros(d, device=dev)
    dx = torch.empty_like(x)
    from ..ops.flash import Positions

    cases = []
    cases.append(("rmsnorm_fwd", lambda: K.rmsnorm_fwd(x, g, 1e-6, out=y, rstd=rstd), 2 * M * d * 2))
    cases.append(("rmsnorm_bwd (+residual)", lambda: K.rmsnorm_bwd(y, x, g, rstd, dw, dres=y, out=dx), 4 * M * d * 2))
    qk = torch.randn(1, M, 2 * H, D, device=dev).to(bf)
    cases.append(("rope (q and k heads, in place)", lambda: K.rope_(qk, Positions(0), 10000.0), 2 * qk.numel() * 2))
    Mc = min(M, 8192)  # the feed-forward and the loss run in chunks of 8192 rows
    gu = torch.randn(Mc, 2 * F, device=dev).to(bf)
    hh = torch.empty(Mc, F, device=dev, dtype=bf)
    cases.append(("swiglu_fwd (8192-row chunk)", lambda: K.swiglu_fwd(gu, out=hh), Mc * 3 * F * 2))
    cases.append(("swiglu_bwd (8192-row chunk)", lambda: K.swiglu_bwd_(gu, hh), Mc * 5 * F * 2))
    table = torch.randn(V, d, device=dev).to(bf)
    tok = torch.randint(0, V, (M,), device=dev, dtype=torch.int32)
    emb = torch.empty(M, d, device=dev, dtype=bf)
    dtab = torch.zeros(V, d, device=dev)
    cases.append(("embedding_fwd", lambda: K.embedding_fwd(tok, table, out=emb), 2 * M * d * 2))
    cases.append(("embedding_bwd (fp32 scatter-add)", lambda: K.embedding_bwd(tok, emb, dtab), M * d * 2 + 2 * M * d * 4))
    logits = torch.randn(Mc, V, device=dev).to(bf)
    tgt = torch.randint(0, V, (Mc,), device=dev, dtype=torch.int32)
    loss = torch.empty(Mc, device=dev)
    cases.append(("xent_fwd_bwd (8192-row chunk, in place)", lambda: K.xent_fwd_bwd_(logits, tgt, 1e-4, loss=loss),
                  2 * Mc * V * 2))
    n = 1 << 28  # 268M parameters per launch (1 GiB of fp32 each for master, moments and gradient)
    p32, m1, m2, gr = [torch.zeros(n, device=dev) for _ in range(4)]
    p16 = torch.empty(n, device=dev, dtype=bf)
    cases.append(("adamw (fp32 master + moments, bf16 copy)",
                  lambda: K.adamw_(p32, m1, m2, gr, p16, step=1, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                                   weight_decay=0.1, decay_end=n), n * (7 * 4 + 2)))
    acc = torch.zeros(1, device=dev)
    cases.append(("sumsq (gradient norm)", lambda: K.sumsq(gr, acc), n * 4))
    f32 = torch.randn(M, d, device=dev)
    cases.append(("cast fp32 -> bf16", lambda: K.cast_f32_to_bf16(f32, emb), M * d * 6))
    for name, fn, nbytes in cases:
        ms_t = time_launches(fn, args.warmup, args.iters, args.flush_l2)
        _lib.check_status()
        print(json.dumps({"kernel": name, "rows": M, "ms": round(ms_t, 4), "algorithmic_gb": round(nbytes / 1e9, 3),
                          "gbs": round(nbytes / ms_t / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms_t / 1e6 / peak_gbs, 3),
                          "denominator": how, "iters": args.iters, "warmup": args.warmup}))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--kernel", required=True, choices=["attn_fwd", "attn_bwd", "gemm", "gemm_dgrad", "gemm_wgrad", "gemm_swiglu", "decode",
                                                 "small_m_linear", "sdpa_fwd", "sdpa_bwd", "memory_bound"])
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
    ap.add_argument("--decode-stages", type=int, default=None, choices=[0, 3, 4],
                    help="decode: depth of the asynchronous-copy ring of the cache rows (default: the library's)")
    ap.add_argument("--splits", type=int, default=0, help="decode: row ranges per (batch, head); 0 = the library's choice")
    ap.add_argument("--q-rows", type=int, default=1, choices=[1, 2, 4, 8],
                    help="decode: query rows per cache row (streams sharing the cache)")
    ap.add_argument("--decode-mma-min-rows", type=int, default=None,
                    help="decode: use the tensor-core kernel from this many query rows (default: the library's)")
    ap.add_argument("--linear-mma-min-rows", type=int, default=None,
                    help="small_m_linear: use the tensor-core kernel from this many rows (default: the library's)")
    ap.add_argument("--prologue", default="none", choices=["none", "rmsnorm", "swiglu"],
                    help="small_m_linear: apply RMSNorm or SwiGLU to the input inside the kernel")
    ap.add_argument("--cache-layout", default="heads", choices=["rows", "heads"],
                    help="decode: (B, S, 2, H, D) rows-major cache or (B, 2, H, S, D) heads-major cache")
    ap.add_argument("--mean-doc-len", type=int, default=0,
                    help="attention kernels: packed documents with geometric lengths of this mean (segment ids); "
                         "-1 = segment ids present but all equal")
    args = ap.parse_args(argv)
    peak_tf, peak_gbs, how = peaks()
    torch.manual_seed(0)
    dev = "cuda"
    res = {"kernel": args.kernel, "denominator": how}
    if args.kernel == "memory_bound":
        return memory_bound_table(args, peak_gbs, how)
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
        q = torch.randn(B, args.q_rows, H, D, device=dev).bfloat16()
        if args.cache_layout == "rows":
            cache = torch.randn(B, S, 2, H, D, device=dev).bfloat16()
            ck, cv = cache[:, :, 0], cache[:, :, 1]
        else:  # every (kv, head) is one contiguous stream of S rows
            cache = torch.randn(B, 2, H, S, D, device=dev).bfloat16()
            ck, cv = cache[:, 0].permute(0, 2, 1, 3), cache[:, 1].permute(0, 2, 1, 3)
        if args.decode_stages is not None:
            Dk.STAGES = args.decode_stages
        if args.decode_mma_min_rows is not None:
            Dk.MMA_MIN_ROWS = args.decode_mma_min_rows
        fn = lambda: Dk.decode_partial(q, ck, cv, q_pos0=S, k_pos0=0, splits=args.splits or None)
        res["cache_layout"] = args.cache_layout
        res["q_rows"] = args.q_rows
        res["tensor_core_kernel"] = args.q_rows >= Dk.MMA_MIN_ROWS
        res["stages"] = Dk.STAGES
        flops = 4.0 * B * S * H * D
        bytes_ = 2.0 * B * S * H * D * 2
        res.update(shape=[B, S, H, D], splits=args.splits or Dk.default_splits(S, B, H, mma=args.q_rows >= Dk.MMA_MIN_ROWS))
    elif args.kernel == "small_m_linear":
        # y[M, N] = x[M, K] W[N, K]^T with M <= 8 (decode-time projections): weight bandwidth is the roofline
        M, N, Kd = min(args.m, 8), args.n, args.k
        ws = [torch.randn(N, Kd, device=dev).bfloat16() for _ in range(8)]  # rotate so that L2 does not help
        x = torch.randn(M, Kd, device=dev).bfloat16()
        turn = [0]

        gain = torch.ones(Kd, device=dev).bfloat16()
        gu = torch.randn(M, 2 * Kd, device=dev).bfloat16()

        def fn():
            turn[0] = (turn[0] + 1) % len(ws)
            if args.prologue == "rmsnorm":  # RMSNorm(x) W^T in one launch
                K.norm_linear(x, gain, 1e-5, ws[turn[0]])
            elif args.prologue == "swiglu":  # (silu(gate) * up) W^T in one launch
                K.swiglu_linear(gu, ws[turn[0]])
            else:
                K.small_m_linear(x, ws[turn[0]])

        if args.linear_mma_min_rows is not None:
            K.LINEAR_MMA_MIN_ROWS = args.linear_mma_min_rows
        res["tensor_core_kernel"] = K._mma_linear_ok(M)
        res["prologue"] = args.prologue

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
        elif args.kernel == "gemm_swiglu":  # h[M,N] = silu(x Wg^T) * (x Wu^T), W = [Wg ; Wu] of 2N rows
            a = torch.randn(M, Kd, device=dev).bfloat16()
            b = (torch.randn(2 * N, Kd, device=dev) * 0.05).bfloat16()
            c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: K.linear_swiglu(a, b, out=c)
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
        flops = 2.0 * M * N * Kd * (2 if args.kernel == "gemm_swiglu" else 1)
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
