"""ctypes binding of the sm_100a kernel library (``_C/libringattn_b200.so``).

The library is built in-tree by :mod:`ringattention_b200._build`. On a machine with a CUDA device
the ops of this package *require* it: :func:`lib` raises if it cannot be loaded, there is no silent
PyTorch fallback on the GPU path. Every launcher returns 0 on success or a negative host error
code; device-side problems (a bounded wait that ran out) are reported through a per-device int32
status word that :func:`check_status` reads.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
_STATUS: dict[int, torch.Tensor] = {}
_LAUNCHES = 0

LIB_PATH = Path(__file__).resolve().parent.parent / "_C" / "libringattn_b200.so"

STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA-filled shared-memory stage",
    2: "timeout waiting for a shared-memory stage to be released",
    3: "timeout waiting for a TMEM accumulator to be produced",
    4: "timeout waiting for a TMEM accumulator to be drained",
    5: "timeout waiting for a peer flag",
    6: "timeout (other)",
    7: "bad argument seen on the device",
}


class KernelError(RuntimeError):
    pass


def available() -> bool:
    """True when the shared object exists (it may still be unusable without a GPU)."""
    return LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library. Unless ``RINGATTN_B200_NO_AUTOBUILD=1``, the incremental build
    runs first (it compares source digests and does nothing when the library is current), so that a stale
    shared object is never used after an edit of the CUDA sources. With ``RINGATTN_B200_BOUNDS_CHECK=1`` the
    checked variant of the library is built and loaded instead."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        from .. import _build

        path = _build.LIB_PATH
        if os.environ.get("RINGATTN_B200_NO_AUTOBUILD") == "1":
            if not path.exists():
                raise KernelError(f"{path} is missing; run python -m ringattention_b200._build")
        else:
            try:
                _build.build()
            except _build.NvccMissing as e:  # an installed wheel on a machine without the toolkit
                if not path.exists():
                    raise KernelError(f"cannot build {path}: {e}") from e
        handle = ctypes.CDLL(str(path))
        handle.ra_last_error.restype = ctypes.c_char_p
        _LIB = handle
    return _LIB


def status_tensor(device: torch.device | int | None = None) -> torch.Tensor:
    """The int32 status word kernels write to on ``device`` (allocated once per device)."""
    if device is None:
        idx = torch.cuda.current_device()
    elif isinstance(device, int):
        idx = device
    else:
        idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _STATUS[idx] = t
    return t


def check_status(device=None, reset: bool = True) -> None:
    """Synchronise and raise :class:`KernelError` if any kernel recorded a failure."""
    t = status_tensor(device)
    code = int(t[0].item())
    if code != 0:
        if reset:
            t.zero_()
        raise KernelError(f"device status {code}: {STATUS_NAMES.get(code, 'unknown')}")


BOUNDS_TAGS = {1: "gemm store", 2: "gemm residual", 10: "attention forward out", 11: "attention forward lse",
               12: "attention forward carry", 13: "attention mask bitmap", 14: "segment ids", 15: "key bias",
               20: "attention backward dK/dV", 21: "attention backward prep", 30: "rmsnorm", 31: "rope",
               32: "swiglu", 33: "embedding token id", 34: "embedding row", 35: "cross-entropy target",
               36: "cross-entropy row", 37: "adamw", 38: "cast", 39: "mask packing", 40: "decode cache row",
               41: "decode merge", 42: "decode mask", 43: "small-M linear", 50: "peer copy"}


def bounds_report(reset: bool = True) -> dict:
    """Violations recorded by the checked build of the library (``RINGATTN_B200_BOUNDS_CHECK=1``): kernels
    range-check the indices behind their global-memory accesses, skip an access that is out of range and count
    it. Returns ``{"checked": bool, "violations": n, "first": {...}}``; synchronises the device."""
    out = (ctypes.c_ulonglong * 4)()
    rc = lib().ra_bounds_report(out, int(reset))
    if rc < 0:
        raise KernelError("ra_bounds_report failed")
    rep = {"checked": rc == 1, "violations": int(out[0]), "first": None}
    if out[0]:
        idx = int(out[2])
        rep["first"] = {"access": BOUNDS_TAGS.get(int(out[1]), str(int(out[1]))),
                        "index": idx - (1 << 64) if idx >= (1 << 63) else idx, "limit": int(out[3])}
    return rep


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def launches() -> int:
    """Number of kernels of this library launched so far in this process."""
    return _LAUNCHES


def count_launch(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def call(name: str, *args, n_kernels: int = 1) -> None:
    """Call launcher ``name``; raise with the library's message on a non-zero return code."""
    fn = getattr(lib(), name)
    rc = fn(*args)
    if rc != 0:
        msg = lib().ra_last_error()
        raise KernelError(f"{name} failed ({rc}): {msg.decode() if msg else ''}")
    count_launch(n_kernels)
