"""The allocation-free backward entry point, called through its exported C symbol.

``ra_attn_bwd_noalloc`` serves hosts that cannot allocate device memory when they need a backward
pass (all HBM already owned by their own pool, a loop that cannot afford cudaMalloc's device-wide
synchronisation, or a C program without PyTorch's allocator). Its temporaries sit in a fixed array
inside the library. The test runs it twice in a row, with different inputs, and compares each result
with the regular path, whose temporaries are PyTorch tensors. The second call finds the first
call's data in the shared array, so it also checks that stale contents are cleared.

This file sorts last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular_path(q, k, v, do, cbs, q_off, k_off):
    from ringattention_b200.ops import flash, kernels as K

    ms = flash.MaskSpec(causal_block_size=cbs, q_pos=flash.Positions(q_off), k_pos=flash.Positions(k_off))
    out, lse = flash.flash_fwd(q, k, v, ms)
    lse2, delta = flash.flash_bwd_prep(out, do, lse)
    B, Sq, H, D = q.shape
    dq_acc = torch.zeros(B, Sq, H, D, device=q.device)
    dk, dv = torch.empty_like(k), torch.empty_like(k)
    flash.flash_bwd(q, k, v, do, lse2, delta, ms, dq_acc, dk, dv)
    dq = torch.empty_like(q)
    K.cast_f32_to_bf16(dq_acc.view(B * Sq, H * D), dq.view(B * Sq, H * D))
    return out, lse, dq, dk, dv


def _no_alloc_path(lib, q, k, v, out, do, lse, cbs, q_off, k_off):
    from ringattention_b200.ops import _lib

    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    # outputs are allocated here, by the caller; the entry point itself allocates nothing
    dq, dk, dv = torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(k, float("nan"))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.ra_attn_bwd_noalloc(p(q), p(k), p(v), p(out), p(do), p(lse), p(dq), p(dk), p(dv),
                                 B, H, Sq, Sk, D, cbs, q_off, k_off,
                                 p(_lib.status_tensor()), _lib.stream_ptr())
    assert rc == 0, lib.ra_last_error()
    return dq, dk, dv


def test_no_alloc_backward_matches_regular_path_twice():
    from ringattention_b200.ops import _lib

    lib = _lib.lib()
    lib.ra_attn_bwd_noalloc.restype = ctypes.c_int
    lib.ra_attn_bwd_noalloc_prepare.restype = ctypes.c_int
    # per-device set-up while memory is still to be had: resolves the array's address, loads the kernels
    assert lib.ra_attn_bwd_noalloc_prepare() == 0, lib.ra_last_error()
    assert lib.ra_attn_bwd_noalloc_prepare() == 0  # idempotent
    torch.manual_seed(0)
    cases = [  # (B, Sq, Sk, H, D, cbs, q_off, k_off): different shapes so stale scratch would show
        (2, 512, 512, 4, 128, 1, 0, 0),
        (1, 300, 640, 2, 64, 1, 340, 0),
        # exactly at both limits (4,194,304 dQ elements, 65,536 rows): lse and delta sit right behind the dQ
        # accumulator in the shared array, so a slip in the carve-up would corrupt one of them
        (1, 8192, 1024, 8, 64, 1, 0, 0),
        (2, 512, 512, 4, 128, 1, 0, 0),
    ]
    for (B, Sq, Sk, H, D, cbs, q_off, k_off) in cases:
        q = torch.randn(B, Sq, H, D, device="cuda").bfloat16()
        k = torch.randn(B, Sk, H, D, device="cuda").bfloat16()
        v = torch.randn(B, Sk, H, D, device="cuda").bfloat16()
        do = torch.randn(B, Sq, H, D, device="cuda").bfloat16()
        out, lse, dq_ref, dk_ref, dv_ref = _regular_path(q, k, v, do, cbs, q_off, k_off)
        dq, dk, dv = _no_alloc_path(lib, q, k, v, out, do, lse, cbs, q_off, k_off)
        torch.cuda.synchronize()
        _lib.check_status()
        for got, want in ((dq, dq_ref), (dk, dk_ref), (dv, dv_ref)):
            assert not torch.isnan(got.float()).any()
            # same tolerance as the kernel tests: 2% of the largest reference entry
            assert (got.float() - want.float()).abs().max() <= 0.02 * want.float().abs().max() + 1e-3


def test_no_alloc_rejects_oversized_problems():
    from ringattention_b200.ops import _lib

    lib = _lib.lib()
    lib.ra_attn_bwd_noalloc.restype = ctypes.c_int
    z = ctypes.c_void_p(0)
    # 1 x 8192 x 32 x 128 = 33.5M dQ elements, far above the 4,194,304 limit: refused before any launch
    rc = lib.ra_attn_bwd_noalloc(z, z, z, z, z, z, z, z, z, 1, 32, 8192, 8192, 128, 1, 0, 0, z, z)
    assert rc != 0
    assert b"too large" in lib.ra_last_error()
    # the row limit alone: 512 x 1 x 128 x 64 is exactly 4,194,304 dQ elements (allowed) but every one of the
    # 65,536 (batch, head) pairs pads its single query row to 128 rows of lse/delta: 8,388,608 > 65,536
    rc = lib.ra_attn_bwd_noalloc(z, z, z, z, z, z, z, z, z, 512, 128, 1, 1, 64, 1, 0, 0, z, z)
    assert rc != 0
    assert b"too large" in lib.ra_last_error()
