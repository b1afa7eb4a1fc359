#!/usr/bin/env python
"""Headline benchmark: LLaMA-7B ring-attention training throughput, 64K tokens per GPU (512K
context on 8 GPUs, sp = #GPUs), bf16 with fp32 master weights and AdamW, blockwise feed-forward,
full remat, synthetic uniform tokens, random-init weights.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3

Rank 0 prints one JSON line. ``value`` is whole-job tokens/s of the device-timed training step
(CUDA events around K steps, barrier + synchronize on both sides, max over ranks); ``e2e`` is the
same metric through ``Trainer.train_step`` including, every step, the pinned host->device copy of
the token shard and the device->host read of the loss. ``--impl reference`` reports whether the
unmodified reference can run here.

The whole run is held to ``--time-budget`` seconds of wall clock (default 600; 0 = no limit). A 512K-token
step on 8 GPUs takes most of a minute, so the requested counts may not fit: the first warm-up step is
timed and the counts are cut in this order: warm-up down to 3, end-to-end steps down to 2, timed steps down
to 3, and only then warm-up below 3 (never below 1). The JSON line reports the counts that actually ran in
``steps`` / ``warmup`` / ``e2e.steps`` and the requested ones in ``steps_requested`` / ``warmup_requested``.
Every step trains on a different batch (a small pool of synthetic batches is cycled).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

T_START = time.perf_counter()

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-7b")
    ap.add_argument("--seq-per-gpu", type=int, default=65536)
    ap.add_argument("--global-batch", type=int, default=1)
    ap.add_argument("--mesh", default=None, help="dp,fsdp,tp,sp (default: sp = #GPUs)")
    ap.add_argument("--layout", default="zigzag", choices=["contiguous", "zigzag"])
    ap.add_argument("--layers", type=int, default=None, help="override layer count (debug only; "
                    "a run with this flag is not the headline config)")
    ap.add_argument("--packed-mean-doc-len", type=int, default=0)
    ap.add_argument("--phase-times", action="store_true",
                    help="also report device milliseconds per phase of a step (measured in the end-to-end steps)")
    ap.add_argument("--time-budget", type=float, default=600.0,
                    help="wall-clock seconds for the whole run, counted from process start (0 = no limit)")
    return ap.parse_args()


def plan_counts(warmup_req: int, steps_req: int, warmup_done: int, step_s: float, remaining_s: float):
    """How many more warm-up steps, timed steps and end-to-end steps fit into ``remaining_s`` seconds at
    ``step_s`` seconds per step. Floors: 3 timed steps, 2 end-to-end steps, 3 warm-up steps in total while
    they fit (1 otherwise); what is left over goes to the timed steps, then to the end-to-end steps (at most
    as many as timed steps), then to the warm-up. Returns ``(more_warmup, timed, e2e)``."""
    steps_req = max(1, steps_req)
    k_min, e_min = min(3, steps_req), min(2, steps_req)
    w_floor = max(0, min(warmup_req, 3) - warmup_done)
    w_rest = max(0, warmup_req - warmup_done)
    if remaining_s == float("inf"):
        return w_rest, steps_req, steps_req
    fit = int(remaining_s / max(step_s, 1e-6))
    w = min(w_floor, max(0, fit - k_min - e_min))
    k, e = k_min, e_min
    left = fit - w - k - e
    if left > 0:
        add = min(left, steps_req - k)
        k, left = k + add, left - add
    if left > 0:
        add = min(left, steps_req - e)
        e, left = e + add, left - add
    if left > 0:
        w += min(left, w_rest - w)
    return w, k, e


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while timing."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args) -> int:
    """The reference is a JAX library. It installs (pure Python, --no-deps) but cannot be imported:
    jax/flax are not on this image and there is no index to get them from."""
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref_dir, "ringattention")):
        why = "baseline/_ref is absent (pip install --no-index --no-deps --target baseline/_ref of the reference was not run)"
    else:
        sys.path.insert(0, ref_dir)
        try:
            import ringattention  # noqa: F401
        except Exception as e:  # ModuleNotFoundError: jax
            why = f"reference installed with --no-deps but import fails: {type(e).__name__}: {e} (no jax/flax wheel offline)"
    if why is None:
        why = "reference imports, but it has no training entry point or model of its own to run this config"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from ringattention_b200.config import LlamaConfig, MeshConfig, TrainConfig
    from ringattention_b200.ops import _lib
    from ringattention_b200.trainer import Trainer, init_distributed
    from ringattention_b200.utils.metrics import device_memory_used_gb

    rank, world, local = init_distributed()
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run",
                  file=sys.stderr)
        return 2
    mesh = args.mesh or f"1,1,1,{world}"
    over = {"layout": args.layout if MeshConfig.parse(mesh).sp > 1 else "contiguous"}
    if args.layers is not None:
        over["n_layers"] = args.layers
    cfg = LlamaConfig.named(args.model, **over)
    sp = MeshConfig.parse(mesh).sp
    seq_len = args.seq_per_gpu * sp
    global_batch = args.global_batch * (world // sp)
    tc = TrainConfig(model=args.model, mesh=mesh, seq_len=seq_len, global_batch=global_batch,
                     packed_mean_doc_len=args.packed_mean_doc_len)
    trainer = Trainer(cfg, tc)
    dev = trainer.device

    # a small pool of synthetic batches, cycled, so that no step repeats the batch of the step before it
    pool = []
    for _ in range(4):
        tk, tg, sg = trainer.make_global_batch()
        pool.append((tk.pin_memory(), tg.pin_memory(), sg))
    seg = pool[0][2]
    if seg is not None:  # packed documents: one document layout for all batches (plans and masks are built once)
        pool = [(tk, torch.where(pool[0][1] < 0, pool[0][1], tg), seg) for tk, tg, _ in pool]
    n_step = [0]

    def next_batch():
        n_step[0] += 1
        return pool[n_step[0] % len(pool)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def agree(x: float) -> float:
        """The same number on every rank (max), so that all ranks run the same number of steps."""
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    budget = args.time_budget if args.time_budget > 0 else float("inf")

    def remaining() -> float:
        # 20 s are kept back for the teardown (process-group shutdown, interpreter exit)
        return budget - (time.perf_counter() - T_START) - 20.0

    # ---- warm-up through the public step (also builds plans, symmetric buffers, allocator pools)
    loss = float("nan")
    warm_done = 0
    step_s = 0.0
    if args.warmup > 0:
        barrier()
        t0 = time.perf_counter()
        loss = trainer.train_step(*next_batch())
        barrier()
        step_s = agree(time.perf_counter() - t0)
        warm_done = 1
    more_w, k_steps, e2e_steps = plan_counts(args.warmup, args.steps, warm_done, step_s, agree(remaining()))
    for _ in range(more_w):
        t0 = time.perf_counter()
        loss = trainer.train_step(*next_batch())
        step_s = time.perf_counter() - t0
        warm_done += 1
    if more_w > 0:  # the later warm-up steps give the better estimate (the first one also allocates and plans)
        barrier()
        _, k_steps, e2e_steps = plan_counts(warm_done, args.steps, warm_done, agree(step_s), agree(remaining()))

    # ---- device-timed steps (inputs resident on the device; a different batch each step)
    dev_pool = []
    for tk, tg, _ in pool:
        a, b = trainer.shard_batch(tk, tg, seg)
        dev_pool.append((a.to(dev).contiguous(), b.to(dev).contiguous()))
    ctx = trainer.context(seg)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    launches0 = _lib.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(k_steps):
        tok_d, tgt_d = dev_pool[i % len(dev_pool)]
        loss_t = trainer.device_step(tok_d, tgt_d, ctx)
    e1.record()
    barrier()
    dev_ms = agree(e0.elapsed_time(e1) / max(1, k_steps))
    launches = (_lib.launches() - launches0)
    _lib.check_status(dev)

    # ---- end-to-end steps through Trainer.train_step (pinned H2D of inputs, D2H of the loss)
    if budget != float("inf"):
        e2e_steps = max(min(2, args.steps), min(e2e_steps, int(agree(remaining()) / max(dev_ms / 1e3, 1e-3))))
    timer = None
    if args.phase_times:
        from ringattention_b200.utils.tracing import PhaseTimer, set_phase_timer

        timer = PhaseTimer()
        set_phase_timer(timer)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        loss = trainer.train_step(*next_batch())
    barrier()
    e2e_ms = agree((time.perf_counter() - t0) * 1e3 / e2e_steps)
    clocks = sampler.stop()
    phases = None
    if timer is not None:
        set_phase_timer(None)
        phases = {k: round(v["ms"] / e2e_steps, 2) for k, v in timer.summary().items()}

    tokens_per_step = global_batch * seq_len
    value = tokens_per_step / (dev_ms / 1e3)
    e2e_value = tokens_per_step / (e2e_ms / 1e3)
    peaks = {}
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    peak_tf = float(peaks.get("bf16_tflops_sustained", 1400.0))
    mfu = trainer.model_flops_per_step() / (dev_ms / 1e3) / (world * peak_tf * 1e12)
    if rank == 0:
        out = {
            "metric": "tokens/sec, LLaMA-7B ring-attention training, 64K tokens/GPU (512K ctx at 8 GPUs)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": k_steps,
            "warmup": warm_done, "steps_requested": args.steps, "warmup_requested": args.warmup,
            "time_budget_s": args.time_budget, "ms_per_step": dev_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform random tokens, random-init weights (std 0.02)",
            "tokens_per_sec_per_gpu": value / world, "mfu_of_measured_sustained_bf16": mfu,
            "loss": loss,
            "config": {"model": args.model, "n_layers": cfg.n_layers, "global_batch": global_batch,
                       "seq_len": seq_len, "parallelism": MeshConfig.parse(mesh).describe(),
                       "layout": cfg.layout, "remat": cfg.remat,
                       "optimizer": "AdamW fp32 master" + (", state sharded over the ring" if trainer.zero is not None else ""),
                       "l2": "working set (13.5 GB bf16 weights + activations) far exceeds the 126 MB L2; no flush needed",
                       "ffn_chunk": cfg.ffn_chunk_size, "loss_chunk": cfg.loss_chunk_size},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": trainer.h2d_bytes_per_step(),
                    "d2h_bytes_per_step": trainer.d2h_bytes_per_step()},
            "gpu_launches": launches, "gpu_launches_per_step": launches / max(1, k_steps),
            "wall_s": time.perf_counter() - T_START,
            "peak_torch_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
            "device_mem_used_gb": device_memory_used_gb(),
            "impl": "ours",
        }
        if phases is not None:
            out["phase_ms_per_step_rank0"] = phases
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
