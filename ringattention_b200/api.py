"""Public API: ``ringattention``, ``blockwise_feedforward``, ``ringattention_inference`` and the
pure-PyTorch ``ringattention_ref`` (the same four names the reference exports,
ringattention/__init__.py:23-27, with ``ringattention_jax`` -> ``ringattention_ref``).

Dispatch (the reference picks an implementation per XLA platform, __init__.py:12-21):

* CUDA bf16 tensors with head_dim 64 or 128 and at most a key bias -> the fused sm_100a kernels.
  On a multi-rank axis KV blocks are pulled from peer memory inside the kernels.
* anything else (CPU, fp32/fp64, a bias with query rows) -> the PyTorch restatement, which rotates
  KV through the axis' communicator (gloo, NCCL or the in-process fake ring).

The GPU path never silently degrades: if the kernel library cannot be loaded the call raises.
"""
from __future__ import annotations

import warnings
from typing import Any, Callable, Optional, Sequence

import torch
import torch.utils.checkpoint

from .config import POLICY_NOTHING_SAVEABLE, BlockwiseKwargs, _policy_name
from .ops import reference as R
from .parallel.mesh import AxisContext, resolve_axis


_WARNED: set = set()


def _warn_fallback(q: torch.Tensor, why: str) -> None:
    """Tell the user, once per reason, that CUDA tensors are being served by the PyTorch restatement."""
    if q.is_cuda and why not in _WARNED:
        _WARNED.add(why)
        warnings.warn(f"ringattention_b200: {why}; this call runs on the PyTorch path, far slower than the "
                      "sm_100a kernels (which take bf16 tensors with head_dim 64 or 128 and at most a key bias)",
                      RuntimeWarning, stacklevel=3)


def _fallback_reason(q: torch.Tensor, attn_bias) -> str:
    if q.dtype != torch.bfloat16:
        return f"dtype {q.dtype} is not bfloat16"
    if q.shape[-1] not in (64, 128):
        return f"head_dim {q.shape[-1]} is not 64 or 128"
    return "attn_bias has query rows (only a key bias (B, 1|H, 1, S_total) is fused)"


def _fused_ok(q: torch.Tensor, attn_bias) -> bool:
    if not q.is_cuda or q.dtype != torch.bfloat16 or q.shape[-1] not in (64, 128):
        return False
    if attn_bias is not None and (attn_bias.dim() != 4 or attn_bias.shape[-2] != 1):
        return False
    return True


def _symm_ring_for(axis: AxisContext, device):
    if axis.size == 1:
        return None
    if axis.symm_ring is None:
        from .parallel.symm import SymmRing

        axis.symm_ring = SymmRing(axis.group, device)
    return axis.symm_ring


def ringattention(q, k, v, attn_bias=None, segment_ids=None, cache_idx=None, axis_name=None,
                  float32_logits: bool = True, blockwise_kwargs=None):
    """Blockwise ring attention over the mesh axis ``axis_name``.

    Arguments follow ringattention/ringattention_jax.py:93 (README.md:20-36):

    ``q, k, v``  per-rank shards ``(B, S_local, H, D)``; rank r owns tokens ``[r*S_local,
    (r+1)*S_local)`` (or the zig-zag chunks when ``blockwise_kwargs["layout"] == "zigzag"``).
    ``attn_bias``  additive, global along keys: ``(B, 1|H, 1|S, S_total)``, or ``None``.
    ``segment_ids``  global ``(B, S_total)`` ints; tokens attend only inside equal ids.
    ``cache_idx``  ``None`` for training; otherwise the global position of the first query on
    *every* rank (q replicated, KV cache sequence-sharded). Taken as an exact token offset.
    ``axis_name``  registered axis name (``"sp"``), a communicator, or ``None`` for one device.
    ``float32_logits``  accepted for compatibility; logits and softmax state are always fp32
    (bf16 x bf16 products are exact in the fp32 accumulator).
    ``blockwise_kwargs``  the reference's dict (see :class:`~ringattention_b200.config.BlockwiseKwargs`).

    Returns ``(B, S_local, H, D)`` in ``v.dtype``; differentiable w.r.t. q, k, v only.
    """
    kw = BlockwiseKwargs.from_any(blockwise_kwargs)
    axis = resolve_axis(axis_name)
    if q.dim() != 4 or k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError("q must be (B,Sq,H,D) and k, v (B,Sk,H,D) with matching B, H, D")
    if _fused_ok(q, attn_bias):
        from .ops import attention as A

        B, Sq, H, D = q.shape
        plan = A.make_plan(axis.rank, axis.size, B, Sq, k.shape[1], H, kw, segment_ids=segment_ids,
                           attn_bias=attn_bias, cache_idx=cache_idx, device=q.device)
        qq, kk, vv = (t if (t.stride(3) == 1 and not any(s % 8 for s in t.stride()[:3])
                             and t.data_ptr() % 16 == 0) else t.contiguous() for t in (q, k, v))
        return A.RingFlashAttention.apply(qq, kk, vv, plan, _symm_ring_for(axis, q.device))
    _warn_fallback(q, _fallback_reason(q, attn_bias))
    return R.RingAttentionRef.apply(q, k, v, attn_bias, segment_ids, cache_idx, axis.comm,
                                    float32_logits, kw)


def ringattention_ref(q, k, v, attn_bias=None, segment_ids=None, cache_idx=None, axis_name=None,
                      float32_logits: bool = True, blockwise_kwargs=None):
    """Same contract as :func:`ringattention`, always on the PyTorch restatement (any device or
    dtype). It is the CPU path, the oracle of the tests and, with NCCL, the rotation baseline."""
    kw = BlockwiseKwargs.from_any(blockwise_kwargs)
    axis = resolve_axis(axis_name)
    return R.RingAttentionRef.apply(q, k, v, attn_bias, segment_ids, cache_idx, axis.comm,
                                    float32_logits, kw)


def ringattention_inference(q, k, v, attn_mask=None, axis_name=None, float32_logits: bool = True):
    """Decoding attention over a sequence-sharded KV cache
    (ringattention/ringattention_inference.py:67-73).

    ``q (B, q_len, H, D)`` is replicated, ``k, v (B, kv_len, H, D)`` are this rank's cache shard and
    ``attn_mask`` is boolean (True = attend), broadcastable to ``(B, H, q_len, S_total)`` and global
    on its last axis. On CUDA bf16 the KV cache stays where it is: every rank computes a partial
    ``(o, lse)`` over its shard (the split-KV decode kernel for up to 8 query rows without gradients, the
    flash-attention kernel with the mask as a bitmap for longer queries or when gradients are needed) and
    the partials are merged through peer memory; all ranks return the same result as the reference's
    rotation. Differentiable w.r.t. q, k, v (ringattention_inference.py:38-64): ``dk``/``dv`` belong to the
    local shard, ``dq`` is the full gradient of the replicated queries on every rank.
    """
    axis = resolve_axis(axis_name)
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128):
        from .ops import inference as Inf

        return Inf.ring_inference_attention(q, k, v, attn_mask, axis, _symm_ring_for(axis, q.device))
    _warn_fallback(q, _fallback_reason(q, None))
    return R.RingAttentionInferenceRef.apply(q, k, v, attn_mask, axis.comm, float32_logits)


def blockwise_feedforward(feedforward: Callable, inputs: torch.Tensor, chunk_size: int,
                          static_argnums: Sequence[int] = (1,), policy: Any = POLICY_NOTHING_SAVEABLE,
                          pre_remat: bool = True, *extra_args):
    """Apply a position-wise ``feedforward`` to ``inputs (B, S, D)`` in chunks of ``chunk_size``
    tokens (ringattention/ringattention_jax.py:333-352).

    Peak activation memory is that of one chunk. With ``pre_remat=False`` each chunk is wrapped in
    activation checkpointing when ``policy`` is ``nothing_saveable`` (the reference wraps with
    ``partitioning.remat``; the default ``pre_remat=True`` assumes the caller already did).
    ``static_argnums`` is accepted for signature compatibility. A
    :class:`~ringattention_b200.ops.ffn.FusedSwiGLU` module as ``feedforward`` runs its chunks on the sm_100a
    GEMM kernels (activation in the GEMM epilogue, per-chunk recomputation in the backward unless ``policy``
    with ``pre_remat=False`` says everything is saveable); any other callable is looped over in PyTorch.
    """
    if inputs.dim() != 3:
        raise ValueError("inputs must be (B, S, D)")
    B, S, D = inputs.shape
    if chunk_size <= 0 or S % chunk_size:
        raise ValueError(f"chunk_size {chunk_size} must divide the sequence length {S}")
    from .ops.ffn import FusedSwiGLU

    if isinstance(feedforward, FusedSwiGLU) and inputs.is_cuda and inputs.dtype == torch.bfloat16:
        # kernel-backed chunk loop with the policy's recomputation built in (a chunk holds chunk_size tokens
        # of every batch row, like one scan step of the reference)
        return feedforward.blockwise(inputs, chunk_size * B if B > 1 else chunk_size,
                                     policy if not pre_remat else POLICY_NOTHING_SAVEABLE)
    remat = (not pre_remat) and _policy_name(policy) == POLICY_NOTHING_SAVEABLE
    outs = []
    for s0 in range(0, S, chunk_size):
        chunk = inputs[:, s0:s0 + chunk_size]
        if remat and torch.is_grad_enabled():
            y = torch.utils.checkpoint.checkpoint(feedforward, chunk, *extra_args, use_reentrant=False)
        else:
            y = feedforward(chunk, *extra_args)
        outs.append(y)
    return torch.cat(outs, dim=1)
