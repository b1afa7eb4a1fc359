#!/usr/bin/env python
"""Long-context inference entry point: chunked prefill into a sequence-sharded KV cache, then
greedy decoding. Reports prefill tokens/s, decode tokens/s and p50 per-token latency as JSON.

    python infer.py --model llama-7b --context 131072 --new-tokens 64
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 infer.py \
        --model llama-7b --context 1048576 --chunk 32768 --new-tokens 256 --batch 1
    ... --streams 4      # four decode streams that share the one cached context
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="llama-7b")
    ap.add_argument("--context", type=int, default=131072, help="tokens of cached context to prefill")
    ap.add_argument("--chunk", type=int, default=32768)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--streams", type=int, default=0,
                    help="decode this many streams (<= 8) from ONE cached context (batch must be 1): the way a batch of "
                         "long-context requests fits when distinct contexts do not")
    ap.add_argument("--layers", type=int, default=None, help="override layer count (debug)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from ringattention_b200.config import LlamaConfig
    from ringattention_b200.models.llama_infer import LlamaInference
    from ringattention_b200.ops import _lib
    from ringattention_b200.parallel.mesh import DeviceMesh
    from ringattention_b200.trainer import init_distributed

    rank, world, local = init_distributed()
    mesh = DeviceMesh(f"1,1,1,{world}")
    over = {} if args.layers is None else {"n_layers": args.layers}
    cfg = LlamaConfig.named(args.model, **over)
    dev = torch.device("cuda", local)
    max_ctx = (args.context + args.new_tokens + 128 * world - 1) // (128 * world) * (128 * world)
    kv_gb = args.batch * max_ctx / world * 2 * cfg.d_model * 2 * cfg.n_layers / 1e9
    free_gb = torch.cuda.mem_get_info(dev)[0] / 1e9
    if kv_gb + cfg.n_params() * 2 / 1e9 > free_gb * 0.95:
        if rank == 0:
            print(json.dumps({"error": "KV cache does not fit", "kv_cache_gb_per_gpu": kv_gb,
                              "free_gb": free_gb, "batch": args.batch, "context": args.context}))
        return 0
    eng = LlamaInference(cfg, max_context=max_ctx, batch=args.batch, device=dev, axis=mesh.axis("sp"),
                         streams=args.streams, max_new_tokens=args.new_tokens + 8)
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab_size, (args.batch, args.context), generator=g)
    gen, timing = eng.generate(prompt.to(dev), args.new_tokens, chunk=args.chunk)
    _lib.check_status(dev)
    lat = timing["decode_ms"]
    # the first steps run eagerly and record the CUDA graph; throughput is quoted on the replayed steps
    steady = lat[3:] if len(lat) > 6 else lat
    t = torch.tensor([timing["prefill_s"], sum(steady) / 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "model": args.model, "n_layers": cfg.n_layers, "n_gpus": world, "batch": args.batch,
            "context": args.context, "chunk": args.chunk, "new_tokens": args.new_tokens,
            "prefill_tokens_per_s": args.batch * args.context / float(t[0]),
            "decode_tokens_per_s": max(args.batch, args.streams) * len(steady) / float(t[1]),
            "streams_sharing_the_context": args.streams,
            "decode_first_steps_ms": [round(x, 3) for x in lat[:3]],
            "decode_p50_ms": statistics.median(steady), "decode_p90_ms": sorted(steady)[int(0.9 * (len(steady) - 1))],
            "kv_cache_gb_per_gpu": kv_gb, "data": "random tokens, random-init weights", "dtype": "bf16"}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
