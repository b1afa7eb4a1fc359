"""Tracing helpers: NVTX ranges around host-side phases and the in-kernel phase timestamps of the
attention backward.

The reference only wraps its two TPU backward launches in ``jax.named_scope``
(ringattention_pallas_tpu.py:1232-1235,1615-1616). Here every phase of a training step can be put
in an NVTX range (visible to any CUDA profiler), and the backward kernel can record SM-clock
timestamps of its pipeline hand-offs for one CTA, which is how the overlap of MMA, softmax and dQ
reduction is measured without a profiler.
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("RINGATTN_B200_NVTX", "0") == "1"


def enable_nvtx(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = on


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range when tracing is enabled (``RINGATTN_B200_NVTX=1`` or :func:`enable_nvtx`)."""
    if _ENABLED and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseTimer:
    """Device time per named phase of a step: a CUDA-event pair on the current stream around every
    ``phase(name)`` region while the timer is installed. ``summary()`` synchronizes and returns the
    milliseconds per phase (summed over the regions) and the number of regions."""

    def __init__(self):
        self._pairs = {}

    def _add(self, name, e0, e1):
        self._pairs.setdefault(name, []).append((e0, e1))

    def summary(self, reset: bool = True) -> dict:
        torch.cuda.synchronize()
        out = {name: {"ms": round(sum(a.elapsed_time(b) for a, b in pairs), 3), "regions": len(pairs)}
               for name, pairs in self._pairs.items()}
        if reset:
            self._pairs = {}
        return out


_TIMER = None


def set_phase_timer(timer: "PhaseTimer | None") -> None:
    """Install (or remove, with ``None``) the timer that :func:`phase` regions report to."""
    global _TIMER
    _TIMER = timer


@contextlib.contextmanager
def phase(name: str):
    """Marks a host-side phase of a step (attention forward, linear layers, gradient reduction, ...):
    an NVTX range when NVTX tracing is on, a CUDA-event pair when a :class:`PhaseTimer` is installed,
    otherwise nothing."""
    t = _TIMER
    if t is None and not _ENABLED:
        yield
        return
    if t is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    with nvtx_range(name):
        yield
    if t is not None:
        e1.record()
        t._add(name, e0, e1)


ROLES = ("mma", "softmax", "drain")
SLOTS = {
    "mma": ("dP issued", "p_ready seen", "ds_ready seen", "iteration issued"),
    "softmax": ("s_full seen", "p_ready arrived", "dp_full seen", "ds_ready arrived"),
    "drain": ("dq_full seen", "dq_empty arrived", "staging done", "-"),
}


class BackwardPhaseTrace:
    """Collect phase timestamps of the first compute CTA of the next attention-backward launches.

    >>> with BackwardPhaseTrace() as tr:
    ...     flash.flash_bwd(...)
    >>> tr.cycles_per_iteration()
    """

    def __init__(self, device=None):
        self.index = torch.cuda.current_device() if device is None else torch.device(device).index
        self.buf = torch.zeros(4, 64, 4, dtype=torch.int64, device=f"cuda:{self.index}")

    def __enter__(self):
        from ..ops import flash

        flash.BWD_TRACE_BUFFERS[self.index] = self.buf  # handed to the backward launches of this device only
        return self

    def __exit__(self, *exc):
        from ..ops import flash

        torch.cuda.synchronize(self.index)
        flash.BWD_TRACE_BUFFERS.pop(self.index, None)
        self.table = self.buf.cpu()
        return False

    def cycles_per_iteration(self, first: int = 8, last: int = 40) -> float:
        t = self.table
        return float(t[0, last, 0] - t[0, first, 0]) / (last - first)

    def rows(self, first: int = 8, count: int = 8):
        t = self.table
        base = int(t[0, first, 0])
        out = []
        for it in range(first, first + count):
            out.append({role: [int(t[r, it, s]) - base for s in range(4)] for r, role in enumerate(ROLES)})
        return out
