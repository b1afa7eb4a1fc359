#!/usr/bin/env python
"""Training entry point.

    python train.py --model llama-7b --mesh 1,1,1,1 --seq-len 65536 --steps 10
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 train.py \
        --model llama-7b --mesh 1,1,1,8 --seq-len 524288 --layout zigzag --steps 10
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 train.py \
        --model llama-7b --mesh 1,2,1,4 --seq-len 131072 --global-batch 2 --packed-mean-doc-len 8192

Synthetic data (uniform random tokens; optionally packed documents with geometric lengths, masked
across documents through segment ids). Prints one JSON line of metrics per step.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="llama-7b")
    ap.add_argument("--mesh", default="1,1,1,1", help="dp,fsdp,tp,sp")
    ap.add_argument("--seq-len", type=int, default=65536, help="global sequence length")
    ap.add_argument("--global-batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--layout", default="contiguous", choices=["contiguous", "zigzag"])
    ap.add_argument("--remat", default="nothing_saveable", choices=["nothing_saveable", "everything_saveable", "save_attention"])
    ap.add_argument("--packed-mean-doc-len", type=int, default=0)
    ap.add_argument("--ckpt-dir", default=None)
    ap.add_argument("--ckpt-every", type=int, default=0)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--log", default=None, help="append JSON lines to this file")
    ap.add_argument("--new-batch-every-step", action="store_true")
    ap.add_argument("--layers", type=int, default=None, help="override the number of layers")
    ap.add_argument("--no-balance", action="store_true",
                    help="packed documents: keep the plain zig-zag pairing instead of the one that balances the documents")
    ap.add_argument("--phase-times", action="store_true",
                    help="log device milliseconds per phase (attention, linear layers, reductions) each step")
    args = ap.parse_args()

    import torch

    from ringattention_b200.config import LlamaConfig, TrainConfig
    from ringattention_b200.trainer import Trainer
    from ringattention_b200.utils.metrics import MetricsLogger, step_metrics
    from ringattention_b200.utils.tracing import PhaseTimer, nvtx_range, set_phase_timer

    over = {} if args.layers is None else {"n_layers": args.layers}
    cfg = LlamaConfig.named(args.model, layout=args.layout, remat=args.remat, **over)
    tc = TrainConfig(model=args.model, mesh=args.mesh, seq_len=args.seq_len, global_batch=args.global_batch,
                     lr=args.lr, steps=args.steps, packed_mean_doc_len=args.packed_mean_doc_len,
                     ckpt_dir=args.ckpt_dir, ckpt_every=args.ckpt_every, resume=args.resume,
                     balance_documents=not args.no_balance)
    tr = Trainer(cfg, tc)
    log = MetricsLogger(args.log, rank=tr.rank)
    if args.resume and args.ckpt_dir:
        tr.load_checkpoint(args.ckpt_dir)
    timer = PhaseTimer() if args.phase_times else None
    set_phase_timer(timer)
    tokens, targets, seg = tr.make_global_batch()
    for _ in range(args.steps):
        if args.new_batch_every_step:
            tokens, targets, seg = tr.make_global_batch()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with nvtx_range("train_step"):
            loss = tr.train_step(tokens, targets, seg)
        ms = (time.perf_counter() - t0) * 1e3
        extra = {} if timer is None else {"phase_ms": {k: v["ms"] for k, v in timer.summary().items()}}
        if timer is not None and getattr(tr.model.params, "shard_count", 1) > 1:
            extra["gather"] = dict(tr.model.params.gather_stats)  # cumulative: gathers, prefetches, resident calls
        log.log(**step_metrics(tr, ms, loss), **extra)
        if args.ckpt_dir and args.ckpt_every and tr.step_idx % args.ckpt_every == 0:
            tr.save_checkpoint(args.ckpt_dir)
    log.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
