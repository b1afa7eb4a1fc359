"""In-tree build of the sm_100a kernel library.

The CUDA sources ship inside the package (``ringattention_b200/csrc``), so an installed wheel can build its
own kernels. Every ``csrc/*.cu`` (plus ``csrc/common/*.cu``) is compiled by ``nvcc`` for ``sm_100a`` only and
linked into ``ringattention_b200/_C/libringattn_b200.so``. The launchers have a C ABI and are bound
from Python with :mod:`ctypes` (see :mod:`ringattention_b200.ops._lib`), so no PyTorch headers are
needed and a full rebuild takes seconds. ``nvcc`` cross-compiles without a GPU.

Run ``python -m ringattention_b200._build`` (``--force`` to rebuild everything, ``-v`` to print the
``ptxas -v`` resource usage).
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "_C"
OBJ_DIR = OUT_DIR / "obj"
LIB_PATH = OUT_DIR / "libringattn_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
    f"-I{CSRC}",
]
# RINGATTN_B200_BOUNDS_CHECK=1 builds the checked variant of the library (libringattn_b200_chk.so): the kernels
# range-check their global-memory indices and record a violation in the status word instead of making the access
BOUNDS_CHECK = os.environ.get("RINGATTN_B200_BOUNDS_CHECK") == "1"
# extra compiler flags (e.g. a -D to try a tuning constant); they are part of the objects' digest
NVCC_FLAGS += os.environ.get("RINGATTN_B200_NVCC_FLAGS", "").split()
if BOUNDS_CHECK:
    NVCC_FLAGS.append("-DRA_BOUNDS_CHECK=1")
    OBJ_DIR = OUT_DIR / "obj_chk"
    LIB_PATH = OUT_DIR / "libringattn_b200_chk.so"


class NvccMissing(RuntimeError):
    """No CUDA compiler on this machine (the prebuilt library, if any, has to do)."""


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise NvccMissing("nvcc not found; the sm_100a kernels cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted((CSRC / "common").glob("*.cu"))


def _headers_digest() -> str:
    h = hashlib.sha1()
    for p in sorted(CSRC.rglob("*.cuh")) + sorted(CSRC.rglob("*.h")):
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(src: Path, hdr_digest: str, force: bool, verbose: bool) -> tuple[Path, bool, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".stamp")
    digest = hashlib.sha1(src.read_bytes() + hdr_digest.encode()).hexdigest()
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, False, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = proc.stdout + proc.stderr
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{log}")
    stamp.write_text(digest)
    (OBJ_DIR / (src.stem + ".ptxas.log")).write_text(log)
    return obj, True, log


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and link the kernel library; returns the path of the shared object."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    # one builder at a time: the ranks of a job all come through here at start-up
    import fcntl

    with open(OBJ_DIR / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        return _build_locked(srcs, force, verbose)


def _build_locked(srcs, force: bool, verbose: bool) -> Path:
    hdr = _headers_digest()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile_one(s, hdr, force, verbose), srcs))
    changed = any(c for _, c, _ in results)
    if verbose:
        for (_, c, log), s in zip(results, srcs):
            if c:
                print(f"--- {s.name}\n{log}")
    if changed or not LIB_PATH.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *[str(o) for o, _, _ in results],
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}{proc.stderr}")
    return LIB_PATH


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    args = ap.parse_args(argv)
    path = build(force=args.force, verbose=args.verbose)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
