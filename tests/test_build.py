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
