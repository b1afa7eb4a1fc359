"""JSON-lines metrics for training and inference runs (the reference has no logging at all)."""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Any, Dict, Optional

import torch


def measured_peaks(repo_root: Optional[str] = None) -> Dict[str, float]:
    """bf16 TFLOP/s and HBM GB/s denominators: ``MEASURED_PEAKS.json`` if present, else the
    fallback figures (1590 TFLOP/s burst, 1400 sustained, 6650 GB/s)."""
    root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class MetricsLogger:
    """Writes one JSON object per line to a file and/or stdout (rank 0 only by default)."""

    def __init__(self, path: Optional[str] = None, echo: bool = True, rank: int = 0):
        self.rank = rank
        self.echo = echo and rank == 0
        self.f = open(path, "a") if (path and rank == 0) else None
        self.t0 = time.time()

    def log(self, **kv: Any) -> None:
        if self.rank != 0:
            return
        kv.setdefault("t", round(time.time() - self.t0, 3))
        line = json.dumps(kv, default=float)
        if self.f:
            self.f.write(line + "\n")
            self.f.flush()
        if self.echo:
            print(line, file=sys.stdout, flush=True)

    def close(self) -> None:
        if self.f:
            self.f.close()


def step_metrics(trainer, step_ms: float, loss: float) -> Dict[str, Any]:
    """tokens/s (whole job and per GPU), MFU against the sustained bf16 peak, peak memory."""
    peaks = measured_peaks()
    toks = trainer.tc.global_batch * trainer.tc.seq_len
    tps = toks / (step_ms / 1e3)
    mfu = trainer.model_flops_per_step() / (step_ms / 1e3) / (trainer.world * peaks["bf16_tflops_sustained"] * 1e12)
    return {"step": trainer.step_idx, "loss": loss, "ms_per_step": step_ms, "tokens_per_s": tps,
            "tokens_per_s_per_gpu": tps / trainer.world, "mfu": mfu, "mfu_denominator": peaks["source"],
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9, "device_mem_used_gb": device_memory_used_gb()}


def device_memory_used_gb() -> float:
    """Bytes of the current device that are in use by anyone, in GB: PyTorch's pools (which keep their peak) plus the
    symmetric buffers this package allocates outside of them."""
    free, total = torch.cuda.mem_get_info()
    return (total - free) / 1e9
