"""Typed Python wrappers over the C launchers (GEMM and the memory-bound driver kernels).

All functions take CUDA tensors, launch on the current stream and return their outputs; they never
fall back to PyTorch math. Shapes follow the LLaMA driver: activations are ``(rows, d)`` bf16.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _lib
from ._lib import ptr, stream_ptr

c_ll = ctypes.c_longlong
c_f = ctypes.c_float


def _status():
    return ptr(_lib.status_tensor())


# ---------------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, group_m: int = 8) -> torch.Tensor:
    """``C[M,N] = A B^T (+ residual)`` on the tcgen05 kernel.

    ``a`` is ``(M, K)`` (``a_mn=False``) or ``(K, M)`` (``a_mn=True``); ``b`` is ``(N, K)`` or
    ``(K, N)``. Both are 2-D bf16 with a contiguous last dim. ``residual`` has C's dtype and may be
    ``out`` itself (in-place accumulation, used for fp32 weight-gradient accumulation).
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"inner dims differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype)
    assert out.shape == (M, N) and out.stride(1) == 1
    c_fp32 = 1 if out.dtype == torch.float32 else 0
    if residual is not None:
        assert residual.dtype == out.dtype and residual.shape == out.shape and residual.stride(1) == 1
    _lib.call("ra_gemm_bf16", ptr(a), ptr(b), ptr(out), ptr(residual), M, N, K,
              c_ll(a.stride(0)), c_ll(b.stride(0)), c_ll(out.stride(0)),
              c_ll(residual.stride(0) if residual is not None else 0),
              int(a_mn), int(b_mn), c_fp32, group_m, _status(), stream_ptr())
    return out


def linear_fwd(x, w, out=None, residual=None):
    """``y = x W^T (+ residual)``; ``x (M,K)``, ``w (N,K)``."""
    return gemm(x, w, out=out, residual=residual)


def linear_swiglu(x, wgu, out=None, group_m: int = 8):
    """``silu(x Wg^T) * (x Wu^T)`` for ``wgu = [Wg ; Wu]`` of shape ``(2F, K)``: the gate/up projection with the
    activation in the GEMM epilogue. ``x (M, K)`` -> ``(M, F)`` bf16."""
    assert x.dtype == torch.bfloat16 and wgu.dtype == torch.bfloat16 and x.dim() == 2 and wgu.dim() == 2
    assert x.stride(1) == 1 and wgu.stride(1) == 1 and wgu.shape[1] == x.shape[1] and wgu.shape[0] % 2 == 0
    M, Kd = x.shape
    F = wgu.shape[0] // 2
    if out is None:
        out = torch.empty(M, F, device=x.device, dtype=torch.bfloat16)
    assert out.shape == (M, F) and out.stride(1) == 1 and out.dtype == torch.bfloat16
    _lib.call("ra_gemm_bf16_swiglu", ptr(x), ptr(wgu), ptr(out), M, F, Kd, c_ll(x.stride(0)),
              c_ll(wgu.stride(0)), c_ll(out.stride(0)), group_m, _status(), stream_ptr())
    return out


def linear_dgrad(dy, w, out=None, residual=None):
    """``dx = dy W (+ residual)``; ``dy (M,N)``, ``w (N,K)`` read MN-major."""
    return gemm(dy, w, b_mn=True, out=out, residual=residual)


def linear_wgrad(dy, x, dw_acc):
    """``dW += dy^T x`` accumulated in fp32; ``dy (M,N)``, ``x (M,K)``, ``dw_acc (N,K)`` fp32."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=dw_acc, residual=dw_acc)


# ---------------------------------------------------------------------------------------------
# normalisation / rope / activation
# ---------------------------------------------------------------------------------------------
def rmsnorm_fwd(x, w, eps: float, out=None, rstd=None):
    rows, d = x.shape
    assert x.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if out is None:
        out = torch.empty_like(x)
    if rstd is None:
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
    _lib.call("ra_rmsnorm_fwd", ptr(x), ptr(w), ptr(out), ptr(rstd), rows, d, c_f(eps), stream_ptr())
    return out, rstd


def rmsnorm_bwd(dy, x, w, rstd, dw_acc, dres=None, out=None):
    """Returns ``dx (+ dres)``; adds the gain gradient to ``dw_acc`` (fp32)."""
    rows, d = x.shape
    assert dy.is_contiguous() and x.is_contiguous() and dw_acc.dtype == torch.float32
    if out is None:
        out = torch.empty_like(x)
    parts = _lib.lib().ra_rmsnorm_bwd_parts(rows)
    scratch = torch.empty(parts, d, device=x.device, dtype=torch.float32)  # per-CTA partial gain gradients
    _lib.call("ra_rmsnorm_bwd", ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(dres), ptr(out), ptr(dw_acc),
              ptr(scratch), rows, d, stream_ptr(), n_kernels=2)
    return out


def rope_(x, positions, theta: float, inverse: bool = False):
    """Rotate a ``(B, S, H, D)`` bf16 view in place. ``positions`` is a flash.Positions map."""
    B, S, H, D = x.shape
    assert x.stride(3) == 1 and x.dtype == torch.bfloat16
    _lib.call("ra_rope", ptr(x), c_ll(x.stride(0)), c_ll(x.stride(1)), c_ll(x.stride(2)), B, S, H, D,
              int(positions.off0), int(positions.off1), int(min(positions.half, 1 << 30)), c_f(theta),
              int(inverse), stream_ptr())
    return x


def swiglu_fwd(gu, out=None):
    rows, f2 = gu.shape
    F = f2 // 2
    assert gu.is_contiguous()
    if out is None:
        out = torch.empty(rows, F, device=gu.device, dtype=torch.bfloat16)
    _lib.call("ra_swiglu_fwd", ptr(gu), ptr(out), c_ll(rows), F, stream_ptr())
    return out


def swiglu_bwd_(gu, dh):
    """Overwrites ``gu`` with ``[d gate | d up]``."""
    rows, f2 = gu.shape
    assert gu.is_contiguous() and dh.is_contiguous()
    _lib.call("ra_swiglu_bwd", ptr(gu), ptr(dh), ptr(gu), c_ll(rows), f2 // 2, stream_ptr())
    return gu


# ---------------------------------------------------------------------------------------------
# embedding / loss
# ---------------------------------------------------------------------------------------------
def embedding_fwd(tokens, table, out=None):
    n = tokens.numel()
    vocab, d = table.shape
    assert tokens.dtype == torch.int32 and tokens.is_contiguous()
    if out is None:
        out = torch.empty(n, d, device=table.device, dtype=torch.bfloat16)
    _lib.call("ra_embedding_fwd", ptr(tokens), ptr(table), ptr(out), c_ll(n), d, vocab, stream_ptr())
    return out


def embedding_bwd(tokens, dy, dtable_acc):
    n = tokens.numel()
    vocab, d = dtable_acc.shape
    assert dtable_acc.dtype == torch.float32 and dy.is_contiguous()
    _lib.call("ra_embedding_bwd", ptr(tokens), ptr(dy), ptr(dtable_acc), c_ll(n), d, vocab, stream_ptr())


def xent_fwd_bwd_(logits, targets, grad_scale: float, loss=None):
    """Per-row loss of a ``(rows, V)`` bf16 logits chunk; the logits are overwritten by
    ``(softmax - onehot) * grad_scale``. Rows whose target is negative get zero loss and gradient."""
    rows, V = logits.shape
    assert logits.stride(1) == 1 and targets.dtype == torch.int32
    if loss is None:
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
    _lib.call("ra_xent_fwd_bwd", ptr(logits), c_ll(logits.stride(0)), ptr(targets), ptr(loss),
              c_ll(rows), V, c_f(grad_scale), stream_ptr())
    return loss


# ---------------------------------------------------------------------------------------------
# optimizer / casts
# ---------------------------------------------------------------------------------------------
def sumsq(g, out):
    """``out[0] += sum(g**2)`` for an fp32 buffer."""
    assert g.dtype == torch.float32 and g.is_contiguous() and out.dtype == torch.float32
    _lib.call("ra_sumsq", ptr(g), c_ll(g.numel()), ptr(out), stream_ptr())
    return out


def adamw_(p, m, v, g, p16, *, step: int, lr: float, beta1: float, beta2: float, eps: float,
           weight_decay: float, decay_end: int, clip: float = 0.0, gnorm_sq=None, grad_mul: float = 1.0):
    """One AdamW step over flat buffers (fp32 master/moments/grads, bf16 working copy)."""
    n = p.numel()
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    _lib.call("ra_adamw", ptr(p), ptr(m), ptr(v), ptr(g), ptr(p16), c_ll(n), c_ll(decay_end),
              c_f(lr), c_f(beta1), c_f(beta2), c_f(eps), c_f(weight_decay), c_f(bc1), c_f(bc2),
              c_f(clip), ptr(gnorm_sq), c_f(grad_mul), stream_ptr())


def cast_f32_to_bf16(src, dst):
    """``src`` ``(rows, d)`` fp32 -> ``dst`` bf16; both 2-D views, row strides allowed."""
    rows, d = src.shape
    assert src.stride(1) == 1 and dst.stride(1) == 1 and dst.shape == src.shape
    _lib.call("ra_cast_f32_bf16", ptr(src), ptr(dst), c_ll(rows), d, c_ll(src.stride(0)),
              c_ll(dst.stride(0)), stream_ptr())
    return dst


def cast_bf16_to_f32(src, dst):
    assert src.is_contiguous() and dst.is_contiguous() and src.numel() == dst.numel()
    _lib.call("ra_cast_bf16_f32", ptr(src), ptr(dst), c_ll(src.numel()), stream_ptr())
    return dst


# From this many rows the small-M products run on the tensor cores (mma.sync with the rows of x as the M side): the
# CUDA-core kernels spend M times the FMAs per weight and fall behind the weight stream.
LINEAR_MMA_MIN_ROWS = int(os.environ.get("RINGATTN_B200_LINEAR_MMA_MIN_ROWS", "2"))


def _mma_linear_ok(M: int) -> bool:
    return LINEAR_MMA_MIN_ROWS <= M <= 8


def _small_m_linear_mma(x, w, residual, out=None):
    M = x.shape[0]
    N, Kd = w.shape
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
    assert out.is_contiguous() and out.shape == (M, N) and x.is_contiguous() and w.is_contiguous()
    assert x.shape[1] == Kd and (residual is None or residual.is_contiguous())
    _lib.call("ra_small_m_linear_mma", ptr(x), ptr(w), ptr(out), ptr(residual), M, N, Kd, stream_ptr())
    return out


def small_m_linear(x, w, out=None, residual=None):
    """``y = x W^T (+ residual)`` for at most 8 rows: a bandwidth-bound kernel that reads every weight
    row once (decode steps). ``x (M,K)``, ``w (N,K)`` bf16 contiguous."""
    M, Kd = x.shape
    N = w.shape[0]
    assert x.is_contiguous() and w.is_contiguous() and M <= 8
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
    assert out.is_contiguous() and (residual is None or residual.is_contiguous())
    if _mma_linear_ok(M):
        return _small_m_linear_mma(x, w, residual, out=out)
    _lib.call("ra_small_m_linear", ptr(x), ptr(w), ptr(out), ptr(residual), M, N, Kd, stream_ptr())
    return out


def _fused_small_m_ok(x, w, residual=None) -> bool:
    """The prologue variant keeps f(x) (rows x K bf16) in shared memory."""
    return (x.shape[0] <= 8 and x.is_contiguous() and w.is_contiguous() and x.dtype == torch.bfloat16
            and (residual is None or residual.is_contiguous())
            and x.shape[0] * w.shape[1] * 2 <= _lib.lib().ra_small_m_linear_fused_max_smem())


def _small_m_linear_fused(x, w, residual, gain, eps, prologue, out=None):
    M = x.shape[0]
    N, Kd = w.shape
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
    assert out.is_contiguous() and out.shape == (M, N)
    _lib.call("ra_small_m_linear_fused", ptr(x), ptr(w), ptr(out), ptr(residual), ptr(gain), c_f(eps), prologue,
              M, N, Kd, stream_ptr())
    return out


def linear_auto(x, w, out=None, residual=None):
    """Pick the tcgen05 GEMM or the small-M kernel by the number of rows."""
    if x.shape[0] <= 8 and x.is_contiguous() and (out is None or out.is_contiguous()) and \
            (residual is None or residual.is_contiguous()):
        return small_m_linear(x, w, out=out, residual=residual)
    return linear_fwd(x, w, out=out, residual=residual)


def norm_linear(x, gain, eps: float, w, out=None):
    """``rmsnorm(x) W^T``. For a handful of rows (decode) the normalisation runs in the prologue of the
    weight-streaming kernel: one launch; otherwise the RMSNorm kernel and the GEMM."""
    assert x.shape[1] == w.shape[1]
    if x.is_contiguous() and x.dtype == torch.bfloat16 and _mma_linear_ok(x.shape[0]):
        h, _ = rmsnorm_fwd(x, gain, eps)  # several rows: the tensor-core kernel takes x as it is
        return _small_m_linear_mma(h, w, None, out=out)
    if _fused_small_m_ok(x, w):
        return _small_m_linear_fused(x, w, None, gain, eps, 1, out=out)
    h, _ = rmsnorm_fwd(x, gain, eps)
    return linear_auto(h, w, out=out)


def swiglu_linear(gu, w, residual=None, out=None):
    """``(silu(gate) * up) W^T (+ residual)`` from the fused gate/up projection ``gu (M, 2F)``; one launch for
    a handful of rows."""
    assert gu.shape[1] == 2 * w.shape[1]
    if gu.is_contiguous() and gu.dtype == torch.bfloat16 and _mma_linear_ok(gu.shape[0]) and \
            (residual is None or residual.is_contiguous()):
        return _small_m_linear_mma(swiglu_fwd(gu), w, residual, out=out)
    if _fused_small_m_ok(gu, w, residual):
        return _small_m_linear_fused(gu, w, residual, None, 0.0, 2, out=out)
    return linear_auto(swiglu_fwd(gu), w, out=out, residual=residual)


def rope_append(qkv, k_cache, v_cache, pos_state, theta: float, k0: int = 0, stripe=None):
    """RoPE of the q and k heads of a one-token ``(B, 1, 3, H, D)`` qkv buffer, in place, at the position in
    ``pos_state[0]``, and the cache append of :func:`kv_append` (rotated K, V), in one launch."""
    B, S_max, H, D = k_cache.shape
    assert qkv.is_contiguous() and qkv.numel() == B * 3 * H * D
    assert k_cache.stride() == v_cache.stride() and k_cache.stride(3) == 1
    sn, sr, sb, sl = stripe if stripe is not None else (0, 0, 0, 0)
    _lib.call("ra_rope_append", ptr(qkv), ptr(k_cache), ptr(v_cache), c_ll(k_cache.stride(0)),
              c_ll(k_cache.stride(1)), c_ll(k_cache.stride(2)), ptr(pos_state), c_f(theta), c_ll(k0), S_max, B, H, D,
              int(sn), int(sr), c_ll(sb), c_ll(sl), stream_ptr())


def rope_at_(x, pos_state, theta: float, offset: int = 0):
    """In-place RoPE of a ``(B, S, H, D)`` view whose first token sits at ``pos_state[0] + offset``,
    with the position read from device memory (decode under a CUDA graph)."""
    B, S, H, D = x.shape
    _lib.call("ra_rope_at", ptr(x), c_ll(x.stride(0)), c_ll(x.stride(1)), c_ll(x.stride(2)), B, S, H, D,
              int(offset), ptr(pos_state), c_f(theta), stream_ptr())
    return x


def kv_append(qkv, k_cache, v_cache, pos_state, k0: int = 0, stripe=None):
    """Write the K/V rows of a one-token ``(B, 1, 3, H, D)`` qkv buffer into the cache shard, given as two
    ``(B, S_max, H, D)`` views of any layout with equal strides, when the position in ``pos_state[0]`` belongs to
    this rank: row ``pos - k0`` of a contiguous shard, or, with ``stripe = (ranks, rank, prefilled rows, prefilled
    positions)``, row ``rows + i // ranks`` on rank ``i % ranks`` for decoded token ``i = pos - positions``."""
    B, S_max, H, D = k_cache.shape
    assert qkv.is_contiguous() and k_cache.stride() == v_cache.stride() and k_cache.stride(3) == 1
    sn, sr, sb, sl = stripe if stripe is not None else (0, 0, 0, 0)
    _lib.call("ra_kv_append", ptr(qkv), ptr(k_cache), ptr(v_cache), c_ll(k_cache.stride(0)), c_ll(k_cache.stride(1)),
              c_ll(k_cache.stride(2)), ptr(pos_state), c_ll(k0), S_max, B, H, D, int(sn), int(sr), c_ll(sb), c_ll(sl),
              stream_ptr())


def decode_advance(state):
    """``state[0] += 1`` (position) and ``state[1] += 1`` (step) on the device."""
    _lib.call("ra_decode_advance", ptr(state), stream_ptr())
