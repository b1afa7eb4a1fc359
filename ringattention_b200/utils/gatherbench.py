"""Benchmark of the GEMM with the FSDP parameter gather inside, on 2+ GPUs (fsdp = number of ranks).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m ringattention_b200.utils.gatherbench --tokens 32768

For the four matrices of one LLaMA-7B layer, forward (``x W^T``, shards along N) and dgrad (``dy W``,
shards along the reduction dimension), it times
* ``plain``    - the ordinary kernel on a fully assembled local copy of the matrix;
* ``resident`` - the sharded kernel when the remote shards are already in the landing area
  (no copy CTAs, every CTA computes);
* ``gather``   - the sharded kernel when this call has to pull the remote shards itself
  (16 copy CTAs; tiles that need remote rows wait for them).
The variants are timed in turn, several rounds, and the minimum is reported (the clock under the
power cap drifts within a run). CUDA events, rank 0's figures.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from ..config import LlamaConfig
from ..models.params import FlatParams
from ..ops import _lib
from ..ops import kernels as K
from ..parallel.mesh import DeviceMesh
from ..trainer import init_distributed


def _time(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=6)
    ap.add_argument("--rounds", type=int, default=4)
    args = ap.parse_args(argv)
    rank, world, local = init_distributed()
    if world < 2:
        print(json.dumps({"error": "needs at least 2 ranks"}))
        return 0
    dev = torch.device("cuda", local)
    mesh = DeviceMesh(f"1,{world},1,1", register=False)
    cfg = LlamaConfig.named("llama-7b", n_layers=1)
    P = FlatParams(cfg, dev, seed=1, with_optimizer=False, shard=(rank, world), fsdp_group=mesh.axis("fsdp").group)
    P.sched.prefetch = False
    M = args.tokens
    for name in ("l0.wqkv", "l0.wo", "l0.wgu", "l0.wd"):
        _, N, Kd, _ = P.mat[name]
        x = torch.randn(M, Kd, device=dev).bfloat16()
        dy = torch.randn(M, N, device=dev).bfloat16()
        w = torch.randn(N, Kd, device=dev).bfloat16()

        def gather_f():
            P.sched.invalidate()
            P.lin_fwd(x, name)

        def gather_d():
            P.sched.invalidate()
            P.lin_dgrad(dy, name)

        fns = {"plain_fwd": lambda: K.linear_fwd(x, w), "resident_fwd": lambda: P.lin_fwd(x, name),
               "plain_dgrad": lambda: K.linear_dgrad(dy, w), "resident_dgrad": lambda: P.lin_dgrad(dy, name)}
        P.lin_fwd(x, name)  # make the shards resident
        best = {k: float("inf") for k in fns}
        for _ in range(args.rounds):
            for k, fn in fns.items():
                best[k] = min(best[k], _time(fn, args.iters))
        best["gather_fwd"] = _time(gather_f, args.iters)
        best["gather_dgrad"] = _time(gather_d, args.iters)
        if rank == 0:
            print(json.dumps({"matrix": name, "shape": [M, N, Kd], "fsdp": world,
                              **{k + "_ms": round(v, 3) for k, v in best.items()},
                              "plain_fwd_tflops": round(2.0 * M * N * Kd / best["plain_fwd"] / 1e9, 1)}), flush=True)
        dist.barrier()
    _lib.check_status(dev)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
