"""Per-GPU memory model of a training step and the maximum trainable context it implies.

    python -m ringattention_b200.utils.memory --model llama-7b --gpus 1 2 4 8

The model mirrors what the driver allocates (``models/params.py``, ``models/llama.py``,
``parallel/symm.py``): bf16 weights, fp32 master + two AdamW moments (sharded over fsdp, and with
``zero1`` also over the sp/dp ranks that hold the same parameters), fp32 gradients (full size), one saved layer input per layer (``nothing_saveable``), the working set of one
layer being recomputed and differentiated, the chunked FFN / LM-head temporaries and, for sp > 1,
the symmetric KV slots, the two local slabs, the fp32 dK/dV accumulator and the fp32 output carry.
Activation memory is linear in the tokens per GPU, so the maximum context grows linearly with the
number of GPUs on the sp axis (the reference's claim, README.md:5). ``inference_max_context`` does the
same for the striped KV cache of the inference engine.
"""
from __future__ import annotations

import argparse
import json

from ..config import LlamaConfig

GiB = 1024 ** 3


def bytes_per_gpu(cfg: LlamaConfig, tokens_per_gpu: int, sp: int = 1, fsdp: int = 1, batch: int = 1,
                  zero1: bool = True, dp: int = 1) -> dict:
    n_mat = cfg.n_layers * (4 * cfg.d_model ** 2 + 3 * cfg.d_model * cfg.d_ff) + cfg.vocab_size * cfg.d_model
    n_rep = cfg.vocab_size * cfg.d_model + (2 * cfg.n_layers + 1) * cfg.d_model
    T = tokens_per_gpu * batch
    d, F, V = cfg.d_model, cfg.d_ff, cfg.vocab_size
    # sharded weights: own shard + the landing area of gathered shards (two regions per kind of matrix)
    landing = 0 if fsdp == 1 else 2 * (fsdp - 1) / fsdp * 2 * (4 * d * d + 3 * F * d + V * d)
    weights = (n_mat / fsdp + n_rep) * 2 + landing
    replicas = sp * dp if zero1 else 1   # ranks that share a parameter shard each keep one slice of its state
    optimizer = (n_mat / fsdp + n_rep) * 12 / replicas
    grads = (n_mat + n_rep) * 4
    saved = cfg.n_layers * T * d * 2
    # one layer in flight (recompute + backward): x2, h1, h2, qkv, attn, dqkv, dattn/dh buffers, dq fp32, lse/delta
    layer = T * d * 2 * (1 + 1 + 1 + 3 + 1 + 3 + 2) + T * d * 4 + 3 * T * cfg.n_heads * 4
    chunks = min(cfg.ffn_chunk_size, T) * (2 * F * 2 + 2 * F * 2) + min(cfg.loss_chunk_size, T) * V * 2
    ring = 0
    if sp > 1:
        kv = T * 2 * d * 2
        ring = 2 * kv + 2 * kv + T * 2 * d * 4 + T * d * 4
    total = weights + optimizer + grads + saved + layer + chunks + ring
    return {"weights": weights, "optimizer": optimizer, "grads": grads, "saved_layer_inputs": saved,
            "layer_working_set": layer, "chunk_temporaries": chunks, "ring_buffers": ring, "total": total}


def max_context(cfg: LlamaConfig, gpus: int, hbm_bytes: float = 178 * GiB, fsdp: int = 1, reserve: float = 0.06,
                zero1: bool = True) -> int:
    """Largest global sequence (multiple of 1024 tokens per GPU) that fits with sp = gpus / fsdp."""
    sp = gpus // fsdp
    lo, hi = 0, 1 << 24
    while hi - lo > 1024:
        mid = (lo + hi) // 2 // 1024 * 1024
        if bytes_per_gpu(cfg, mid, sp, fsdp, zero1=zero1)["total"] <= hbm_bytes * (1 - reserve):
            lo = mid
        else:
            hi = mid
    return lo * sp


def inference_max_context(cfg: LlamaConfig, gpus: int, batch: int = 1, chunk: int = 32768,
                          hbm_bytes: float = 178 * GiB, reserve: float = 0.06) -> int:
    """Longest context per sequence (multiple of 128 * gpus) whose striped KV cache fits beside the
    replicated bf16 weights and the working set of one prefill chunk (``models/llama_infer.py``)."""
    d, F, V = cfg.d_model, cfg.d_ff, cfg.vocab_size
    n_par = cfg.n_layers * (4 * d * d + 3 * d * F) + 2 * V * d
    t = chunk // gpus
    # per chunk: gathered queries + fp32 partials and their exchange buffers (x3), local qkv, ffn chunk
    work = batch * (chunk * d * (2 + 3 * 4) + t * d * 2 * 8 + min(cfg.ffn_chunk_size, t) * 3 * F * 2)
    free = hbm_bytes * (1 - reserve) - n_par * 2 - work
    per_token = 2 * d * 2 * cfg.n_layers / gpus * batch          # K and V, bf16, all layers, this GPU's share
    ctx = int(free / per_token)
    return max(0, ctx // (128 * gpus) * (128 * gpus))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="llama-7b")
    ap.add_argument("--gpus", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--fsdp", type=int, default=1)
    ap.add_argument("--no-zero1", action="store_true", help="optimizer state replicated over sp (as before zero1)")
    ap.add_argument("--inference-batch", type=int, default=0,
                    help="also print the longest inference context for this batch size")
    args = ap.parse_args(argv)
    cfg = LlamaConfig.named(args.model)
    for g in args.gpus:
        ctx = max_context(cfg, g, fsdp=args.fsdp, zero1=not args.no_zero1)
        b = bytes_per_gpu(cfg, ctx // max(1, g // args.fsdp), g // args.fsdp, args.fsdp, zero1=not args.no_zero1)
        print(json.dumps({"gpus": g, "fsdp": args.fsdp, "max_context_tokens": ctx,
                          "gib_per_gpu": {k: round(v / GiB, 1) for k, v in b.items()}}))
        if args.inference_batch:
            print(json.dumps({"gpus": g, "inference_batch": args.inference_batch,
                              "max_inference_context_tokens": inference_max_context(cfg, g, args.inference_batch)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
