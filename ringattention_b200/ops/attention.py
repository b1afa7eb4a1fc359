"""Ring attention on the sm_100a kernels: planning, forward, backward, autograd binding.

A :class:`RingPlan` fixes, for this rank, which KV block is visited at every ring step and the
masks that apply (global positions, segment ids, key bias, dropout seed). The forward visits block
``(rank - t) mod N`` at step ``t`` like the reference (ringattention_jax.py:36), but KV never
rotates: the block is *pulled* straight from its owner's memory over NVLink by copy CTAs inside the
attention kernel of the previous step into a double-buffered local slab, and the carry is merged
in the kernel epilogue. Steps whose block is entirely in the causal future are skipped (the
reference still rotates through them, ringattention_jax.py:147-164,47). The backward pulls K/V the
same way and returns dK/dV to the owner with fp32 reductions from the kernel epilogue.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..config import BlockwiseKwargs
from . import flash
from . import kernels as K
from .flash import MaskSpec, Positions
from .reference import shard_segments
from ..utils.tracing import phase


@dataclass
class RingStep:
    block: int            # owner rank of the KV block
    mask: MaskSpec
    needed: bool = True   # False when the causal rule hides the whole block


@dataclass
class RingPlan:
    rank: int
    world: int
    steps: List[RingStep] = field(default_factory=list)

    @property
    def active(self) -> List[RingStep]:
        return [s for s in self.steps if s.needed]


def _block_needed(q_segs, k_segs, cbs: Optional[int]) -> bool:
    if not cbs:
        return True
    q_hi = max(g + n - 1 for _, g, n in q_segs)
    k_lo = min(g for _, g, _ in k_segs)
    return q_hi // cbs >= k_lo // cbs


def make_plan(rank: int, world: int, B: int, Sq: int, Sk: int, H: int, kw: BlockwiseKwargs, *,
              segment_ids: Optional[torch.Tensor] = None, attn_bias: Optional[torch.Tensor] = None,
              cache_idx: Optional[int] = None, device=None) -> RingPlan:
    """Build the per-step masks. ``segment_ids`` is global ``(B, S_total)``; ``attn_bias`` is a key
    bias ``(B, 1|H, 1, S_total)`` (global along keys, README.md:43)."""
    layout = kw.layout if cache_idx is None else "contiguous"
    if cache_idx is None:
        q_segs = shard_segments(rank, world, Sq, layout)
    else:
        q_segs = [(0, int(cache_idx), Sq)]
    q_pos = Positions.from_segments(q_segs)
    cbs = int(kw.causal_block_size) if kw.causal_block_size else 0
    seed = kw.seed()
    pdrop = float(kw.attn_pdrop) if kw.dropout_active else 0.0
    seg_q = seg_q_mm = None
    if segment_ids is not None:
        seg32 = segment_ids.to(device=device, dtype=torch.int32)
        seg_q = seg32.index_select(1, q_pos.tensor(Sq, device)).contiguous()
        seg_q_mm = flash.seg_tile_minmax(seg_q)
    if attn_bias is not None:
        if attn_bias.dim() != 4 or attn_bias.shape[-2] != 1:
            raise NotImplementedError(
                "the fused kernels take a key bias of shape (B, 1|H, 1, S_total); a bias with query "
                "rows is served by the PyTorch path (ringattention_b200.ops.reference)")
        bias_f = attn_bias.to(device=device, dtype=torch.float32)[:, :, 0, :]
    plan = RingPlan(rank=rank, world=world)
    for t in range(world):
        j = (rank - t) % world
        k_segs = shard_segments(j, world, Sk, layout)
        k_pos = Positions.from_segments(k_segs)
        ms = MaskSpec(causal_block_size=cbs, q_pos=q_pos, k_pos=k_pos, seed=seed, pdrop=pdrop)
        if segment_ids is not None:
            ms.seg_q, ms.seg_q_mm = seg_q, seg_q_mm
            ms.seg_k = seg32.index_select(1, k_pos.tensor(Sk, device)).contiguous()
            ms.seg_k_mm = flash.seg_tile_minmax(ms.seg_k)
        if attn_bias is not None:
            ms.bias = bias_f.index_select(2, k_pos.tensor(Sk, device)).contiguous()
        plan.steps.append(RingStep(block=j, mask=ms, needed=_block_needed(q_segs, k_segs, cbs)))
    return plan


# ---------------------------------------------------------------------------------------------
# forward / backward over a plan
# ---------------------------------------------------------------------------------------------
def ring_forward(q, k, v, plan: RingPlan, symm_ring=None, out=None):
    """Returns ``(out bf16 (B,Sq,H,D), lse fp32 (B,H,Sq))``."""
    if plan.world == 1:
        return flash.flash_fwd(q, k, v, plan.steps[0].mask, out=out)
    if symm_ring is None:
        raise RuntimeError("a multi-rank plan on CUDA needs a symmetric-memory ring "
                           "(ringattention_b200.parallel.symm.SymmRing)")
    return symm_ring.forward(q, k, v, plan, out=out)


def ring_backward(q, k, v, out, lse, dout, plan: RingPlan, symm_ring=None, dq=None, dk=None, dv=None):
    """Returns ``(dq, dk, dv)`` bf16. ``dq/dk/dv`` may be given as (strided) destination views."""
    B, Sq, H, D = q.shape
    with phase("attn_bwd_prep"):
        lse2, delta = flash.flash_bwd_prep(out, dout, lse)
        dq_acc = torch.zeros(B, Sq, H, D, device=q.device, dtype=torch.float32)
    if dk is None:
        dk = torch.empty_like(k)
    if dv is None:
        dv = torch.empty(dk.shape, device=dk.device, dtype=dk.dtype) if dk.is_contiguous() \
            else torch.empty_strided(dk.shape, dk.stride(), device=dk.device, dtype=dk.dtype)
    if plan.world == 1:
        flash.flash_bwd(q, k, v, dout, lse2, delta, plan.steps[0].mask, dq_acc, dk, dv,
                        flash.DKV_STORE_BF16)
    else:
        if symm_ring is None:
            raise RuntimeError("a multi-rank plan on CUDA needs a symmetric-memory ring")
        symm_ring.backward(q, k, v, dout, lse2, delta, plan, dq_acc, dk, dv)
    if dq is None:
        dq = torch.empty_like(q)
    Sd = dq.stride()
    with phase("attn_bwd_dq_cast"):
        _cast_dq(dq_acc, dq, B, Sq, H, D, Sd)
    return dq, dk, dv


def _cast_dq(dq_acc, dq, B, Sq, H, D, Sd):
    if dq.is_contiguous():
        K.cast_f32_to_bf16(dq_acc.view(B * Sq, H * D), dq.view(B * Sq, H * D))
    elif Sd[3] == 1 and Sd[2] == D and Sd[0] == Sq * Sd[1]:
        K.cast_f32_to_bf16(dq_acc.view(B * Sq, H * D), dq.as_strided((B * Sq, H * D), (Sd[1], 1), dq.storage_offset()))
    else:
        dq.copy_(dq_acc)


class RingFlashAttention(torch.autograd.Function):
    """``ringattention`` on CUDA bf16 inputs. Gradients flow to q, k, v only, like the reference
    (ringattention_jax.py:90)."""

    @staticmethod
    def forward(ctx, q, k, v, plan, symm_ring):
        out, lse = ring_forward(q, k, v, plan, symm_ring)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.plan = plan
        ctx.symm_ring = symm_ring
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        if dout.stride(3) != 1 or any(s % 8 for s in dout.stride()[:3]):
            dout = dout.contiguous()
        dq, dk, dv = ring_backward(q, k, v, out, lse, dout, ctx.plan, ctx.symm_ring)
        return dq, dk, dv, None, None
