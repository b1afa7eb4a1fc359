"""The kernel library builds for sm_100a without a GPU and exports its C entry points."""
import ctypes
import shutil

import pytest


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not installed")
def test_build_and_symbols():
    from ringattention_b200 import _build

    path = _build.build()
    assert path.exists()
    lib = ctypes.CDLL(str(path))
    for sym in ("ra_gemm_bf16", "ra_attn_fwd", "ra_attn_bwd", "ra_attn_bwd_prep", "ra_rmsnorm_fwd",
                "ra_rmsnorm_bwd", "ra_rope", "ra_swiglu_fwd", "ra_swiglu_bwd", "ra_xent_fwd_bwd",
                "ra_adamw", "ra_symm_barrier", "ra_peer_copy", "ra_last_error"):
        assert hasattr(lib, sym), sym
    flags = " ".join(_build.NVCC_FLAGS)
    assert "compute_100a" in flags and "sm_100a" in flags


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="nvcc not installed")
def test_wheel_is_self_contained(tmp_path):
    """A wheel built from the tree, installed elsewhere, carries the kernel sources and the compiled library and
    loads it without the source tree."""
    import os
    import subprocess
    import sys

    src = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    # build from a copy, so that setuptools leaves its build/ and egg-info directories outside the repository
    # (the object files travel with the copy: nothing is recompiled)
    repo = str(tmp_path / "src")
    os.makedirs(repo)
    shutil.copytree(os.path.join(src, "ringattention_b200"), os.path.join(repo, "ringattention_b200"),
                    ignore=shutil.ignore_patterns("__pycache__"))
    for f in ("pyproject.toml", "setup.py", "README.md"):
        shutil.copy(os.path.join(src, f), repo)
    dist, site = tmp_path / "dist", tmp_path / "site"
    r = subprocess.run([sys.executable, "-m", "pip", "wheel", "--no-deps", "--no-build-isolation", "--no-index",
                        "-w", str(dist), repo], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    whl = next(dist.glob("ringattention_b200-*.whl"))
    r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-deps", "--no-index", "--target", str(site),
                        str(whl)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert (site / "ringattention_b200" / "csrc" / "attn_fwd_sm100.cu").exists()
    code = ("import ctypes, ringattention_b200.ops._lib as L; "
            f"assert str(L.LIB_PATH).startswith({str(site)!r}), L.LIB_PATH; "
            "h = ctypes.CDLL(str(L.LIB_PATH)); assert hasattr(h, 'ra_attn_fwd'); print('ok')")
    env = dict(os.environ, PYTHONPATH=str(site), RINGATTN_B200_NO_AUTOBUILD="1")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=str(tmp_path))
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
