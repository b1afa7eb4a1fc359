"""Ring-attention operator benchmark on 1/2/4/8 GPUs (sp = number of ranks).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m ringattention_b200.utils.ringbench --tokens-per-gpu 32768 --heads 32 --head-dim 128

Batch 1, bf16, causal, q/k/v ~ N(0,1). Every timing is on the device (CUDA events around the
timed launches, barrier + synchronize on both sides) and the maximum over ranks is reported.

Reported per direction and for forward+backward:
* ``fused``      - the product path: KV pulled from peer memory inside the attention kernels;
* ``no_comm``    - the same kernels on the same blocks with the remote KV already resident in local
  memory (no transfers, staging or barriers): the compute-only time;
* ``serial_copy``- the fused schedule with every pull done by a separate copy kernel before its step,
  i.e. nothing overlapped; ``hidden = (serial - fused) / (serial - no_comm)`` is the fraction of
  the communication cost that the in-kernel pull hides;
* ``rotation``   - (optional, ``--baseline``) the reference algorithm restated in PyTorch: einsum
  blockwise attention with NCCL send/recv rotation of K/V (and dK/dV), the baseline, at a reduced
  size if requested with ``--baseline-tokens-per-gpu``.
Roofline: time >= max(FLOPs / measured bf16 peak, NVLink bytes / 770 GB/s); the achieved fraction
is that bound divided by the measured time, for the slowest rank (most visible blocks).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from ..config import BlockwiseKwargs
from ..ops import _lib, attention as A, flash
from ..ops import reference as R
from ..parallel.mesh import DeviceMesh
from ..parallel.symm import SymmRing, peer_bandwidth_probe
from ..trainer import init_distributed
from .metrics import measured_peaks

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction (GB/s), B200 over NVSwitch


def _timed(fn, warmup, iters, world):
    for _ in range(warmup):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


class _LocalRing:
    """Stand-in for SymmRing whose 'peer' blocks are local copies: same kernels, same blocks, no
    NVLink traffic and no barriers. Gives the compute-only time of the ring schedule."""

    def __init__(self, blocks_k, blocks_v, rank, sync=None):
        """``sync``: a SymmRing whose barriers are kept (one before the forward, one on either side of the
        backward, like the fused schedule), so that the skew between the ranks is in both timings and their
        difference is the cost of moving the data."""
        self.k, self.v, self.rank, self.sync = blocks_k, blocks_v, rank, sync

    def forward(self, q, k, v, plan, out=None):
        if self.sync is not None:
            self.sync.barrier()
        steps = plan.active
        B, Sq, H, D = q.shape
        out = torch.empty(B, Sq, H, D, device=q.device, dtype=torch.bfloat16) if out is None else out
        lse = torch.empty(B, H, Sq, device=q.device, dtype=torch.float32)
        o_acc = torch.empty(B, Sq, H, D, device=q.device, dtype=torch.float32) if len(steps) > 1 else None
        prev = False
        for i, st in enumerate(steps):
            last = i == len(steps) - 1
            flash.flash_fwd(q, self.k[st.block], self.v[st.block], st.mask, o_prev=o_acc if prev else None,
                            lse_prev=lse if prev else None, out=out if last else o_acc, lse_out=lse)
            prev = True
        return out, lse

    def backward(self, q, k, v, dout, lse2, delta, plan, dq_acc, dk, dv):
        acc = {j: (torch.zeros_like(self.k[j], dtype=torch.float32), torch.zeros_like(self.k[j], dtype=torch.float32))
               for j in {s.block for s in plan.active}}
        if self.sync is not None:
            self.sync.barrier()
        for st in plan.active:
            a, b = acc[st.block]
            flash.flash_bwd(q, self.k[st.block], self.v[st.block], dout, lse2, delta, st.mask, dq_acc, a, b,
                            flash.DKV_REDUCE_FP32)
        if self.sync is not None:
            self.sync.barrier()
        dk.copy_(acc[self.rank][0])
        dv.copy_(acc[self.rank][1])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--tokens-per-gpu", type=int, default=32768)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--layout", default="zigzag", choices=["contiguous", "zigzag"])
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--baseline", action="store_true")
    ap.add_argument("--baseline-tokens-per-gpu", type=int, default=0)
    args = ap.parse_args(argv)
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    mesh = DeviceMesh(f"1,1,1,{world}")
    ring = SymmRing(mesh.axis("sp").group, dev) if world > 1 else None
    B, S, H, D = 1, args.tokens_per_gpu, args.heads, args.head_dim
    layout = args.layout if world > 1 else "contiguous"
    torch.manual_seed(rank)
    q, k, v, do = [torch.randn(B, S, H, D, device=dev).bfloat16() for _ in range(4)]
    kw = BlockwiseKwargs(causal_block_size=1, query_chunk_size=2048, key_chunk_size=2048, layout=layout)
    plan = A.make_plan(rank, world, B, S, S, H, kw, device=dev)
    state = {}

    def fwd(r):
        state["out"], state["lse"] = A.ring_forward(q, k, v, plan, r)

    def bwd(r):
        A.ring_backward(q, k, v, state["out"], state["lse"], do, plan, r)

    res = {"n_gpus": world, "tokens_per_gpu": S, "heads": H, "head_dim": D, "layout": layout, "dtype": "bf16",
           "causal": True, "iters": args.iters, "warmup": args.warmup}
    t_f = _timed(lambda: fwd(ring), args.warmup, args.iters, world)
    t_b = _timed(lambda: bwd(ring), args.warmup, args.iters, world)
    res["fused_ms"] = {"fwd": t_f, "bwd": t_b, "fwd_bwd": t_f + t_b}
    _lib.check_status(dev)
    # FLOPs of the slowest rank: visible (q, k) pairs * 4*D (fwd) / 10*D (bwd)
    tot = S * world
    if layout == "zigzag" or world == 1:
        pairs = tot * (tot + 1) / 2 / world                      # balanced
    else:
        pairs = S * S * (world - 1) + S * (S + 1) / 2            # last rank of a contiguous layout
    f_flops, b_flops = 4.0 * pairs * H * D, 10.0 * pairs * H * D
    peaks = measured_peaks()
    res["tflops_per_gpu"] = {"fwd": f_flops / t_f / 1e9, "bwd": b_flops / t_b / 1e9,
                             "fwd_bwd": (f_flops + b_flops) / (t_f + t_b) / 1e9}
    kv_bytes = 2 * S * H * D * 2
    n_remote = len([s for s in plan.active if s.block != rank])
    link_f = n_remote * kv_bytes / (NVLINK_GBS * 1e6)                       # ms, forward pulls
    link_b = n_remote * (kv_bytes + 2 * S * H * D * 4) / (NVLINK_GBS * 1e6)  # pulls + fp32 dK/dV reductions
    bound_f = max(f_flops / (peaks["bf16_tflops"] * 1e9), link_f)
    bound_b = max(b_flops / (peaks["bf16_tflops"] * 1e9), link_b)
    res["roofline"] = {"denominator": peaks["source"], "bound_ms": {"fwd": bound_f, "bwd": bound_b},
                       "fraction": {"fwd": bound_f / t_f, "bwd": bound_b / t_b,
                                    "fwd_bwd": (bound_f + bound_b) / (t_f + t_b)},
                       "nvlink_ms_if_serial": {"fwd": link_f, "bwd": link_b}}
    if world > 1:
        # compute-only variant: fetch the remote blocks once, outside the timed region
        ks, vs = {rank: k}, {rank: v}
        gk = [torch.empty_like(k) for _ in range(world)]
        gv = [torch.empty_like(v) for _ in range(world)]
        dist.all_gather(gk, k.contiguous())
        dist.all_gather(gv, v.contiguous())
        for j in {s.block for s in plan.active}:
            ks[j], vs[j] = gk[j], gv[j]
        local = _LocalRing(ks, vs, rank)
        u_f = _timed(lambda: fwd(local), args.warmup, args.iters, world)
        u_b = _timed(lambda: bwd(local), args.warmup, args.iters, world)
        res["no_comm_no_barrier_ms"] = {"fwd": u_f, "bwd": u_b}
        local = _LocalRing(ks, vs, rank, sync=ring)   # same kernels on resident blocks, same barriers as the fused run
        c_f = _timed(lambda: fwd(local), args.warmup, args.iters, world)
        c_b = _timed(lambda: bwd(local), args.warmup, args.iters, world)
        res["no_comm_ms"] = {"fwd": c_f, "bwd": c_b}
        # the same schedule with every pull done by a separate copy kernel before its step (no overlap)
        ring.overlap = False
        s_f = _timed(lambda: fwd(ring), args.warmup, args.iters, world)
        s_b = _timed(lambda: bwd(ring), args.warmup, args.iters, world)
        ring.overlap = True
        res["serial_copy_ms"] = {"fwd": s_f, "bwd": s_b}
        # what the forward pulls and the backward pulls + fp32 dK/dV reductions would cost back to back at the
        # measured link bandwidth, and how much of that the fused schedule leaves exposed
        res["kv_transfer_hidden"] = {"fwd": 1.0 - max(0.0, t_f - c_f) / max(link_f, 1e-9),
                                     "bwd": 1.0 - max(0.0, t_b - c_b) / max(link_b, 1e-9),
                                     "definition": "1 - (fused - no_comm) / (bytes over NVLink / 770 GB/s)"}
        res["kv_transfer_hidden_vs_serial_copy"] = {
            "fwd": (s_f - t_f) / max(s_f - c_f, 1e-9), "bwd": (s_b - t_b) / max(s_b - c_b, 1e-9),
            "definition": "(serial - fused) / (serial - no_comm); the serial run moves K/V with separate copy kernels"}
        res["comm_overhead_fraction"] = {"fwd": (t_f - c_f) / t_f, "bwd": (t_b - c_b) / t_b}
        res["nvlink_probe"] = peer_bandwidth_probe(ring, nbytes=1 << 28, ctas=64)
        del gk, gv, local, ks, vs
    if args.baseline:
        Sb = args.baseline_tokens_per_gpu or S
        comm = mesh.axis("sp").comm
        qb, kb, vb, dob = [t[:, :Sb].contiguous() for t in (q, k, v, do)]
        kwb = BlockwiseKwargs(causal_block_size=1, query_chunk_size=min(2048, Sb), key_chunk_size=min(2048, Sb))

        def base():
            qq, kk, vv = [t.detach().requires_grad_(True) for t in (qb, kb, vb)]
            o = R.RingAttentionRef.apply(qq, kk, vv, None, None, None, comm, True, kwb)
            o.backward(dob)

        t_base = _timed(base, 1, 1, world)
        pairs_b = Sb * Sb * (world - 1) + Sb * (Sb + 1) / 2
        res["rotation_baseline"] = {"tokens_per_gpu": Sb, "fwd_bwd_ms": t_base,
                                    "tflops_per_gpu": 14.0 * pairs_b * H * D / t_base / 1e9,
                                    "note": "PyTorch restatement of the reference algorithm, NCCL send/recv, contiguous layout"}
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
