"""``ringattention_inference`` on the sm_100a kernels, for any query length and with gradients.

The reference op (ringattention/ringattention_inference.py:8-35) takes replicated queries
``(B, q_len, H, D)``, a sequence-sharded KV cache and a boolean mask that is global along the keys, and
rotates the whole cache around the ring; its VJP (:38-64) rotates K, V, dK and dV once more. Here the
cache never moves:

* forward: every rank runs the flash-attention kernel of its queries against its own shard, with the mask
  slice of that shard packed into a bitmap, and gets a partial ``(o, lse)``. The partials are stored into
  every peer's inbox through peer memory, and each rank merges the N partials (log-sum-exp weights) into
  the same result the rotation would have produced. Up to 8 query rows without gradients take the split-KV
  decode kernel instead (``ops/decode.py``), which streams the cache at HBM speed.
* backward: the five-GEMM kernel runs against the local shard with the merged ``lse``: ``dK``/``dV`` of the
  shard are complete as they are (no other rank holds these keys), and the per-rank ``dQ`` contributions
  are summed over the ring, so every rank returns the full ``dQ`` of its replicated queries, like the
  reference (:61-64).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import decode as Dk
from . import flash
from . import kernels as K
from .flash import MaskSpec, Positions


def _local_mask(attn_mask: Optional[torch.Tensor], rank: int, S_loc: int, B: int, H: int, ql: int):
    """Slice the global boolean mask to this rank's keys and give it query rows: ``(B|1, H|1, ql, S_loc)``."""
    if attn_mask is None:
        return None
    m = attn_mask
    while m.dim() < 4:
        m = m.unsqueeze(0)
    m = m[..., rank * S_loc:(rank + 1) * S_loc]
    if m.shape[-1] != S_loc:
        raise ValueError("attn_mask is too short along the keys: its last axis is global (all shards)")
    if m.shape[2] == 1 and ql > 1:
        m = m.expand(m.shape[0], m.shape[1], ql, S_loc)
    if m.shape[0] == 1 and B > 1:
        m = m.expand(B, *m.shape[1:])
    if m.shape[1] not in (1, H):
        raise ValueError("attn_mask must broadcast to (B, H, q_len, S_total)")
    return m


def _exchange_and_merge(o_p, lse_p, axis, symm_ring):
    """``o_p (B, ql, H, D)`` fp32 and ``lse_p (B, H, ql)``: this rank's partial. Returns the merged
    ``(out bf16 (B, ql, H, D), lse (B, H, ql))``, identical on every rank. The partials travel as peer stores
    into slot ``rank`` of every rank's inbox; a flag barrier orders them before the merge."""
    B, ql, H, D = o_p.shape
    rank, world = axis.rank, axis.size
    rows = B * ql * H
    lse_rows = lse_p.permute(0, 2, 1).contiguous()                      # rows in (b, i, h) order, like o_p
    inbox_o = symm_ring.buffer("infer_inbox_o", 2 * rows * world * D * 4)
    inbox_l = symm_ring.buffer("infer_inbox_lse", 2 * rows * world * 4)
    o_tab, l_tab = symm_ring.peer_ptr_table("infer_inbox_o"), symm_ring.peer_ptr_table("infer_inbox_lse")
    n_o, n_l = rows * world * D, rows * world
    slot = symm_ring.calls & 1                                          # double-buffered across calls
    symm_ring.calls += 1
    o_ptrs = o_tab + slot * n_o * 4
    l_ptrs = l_tab + slot * n_l * 4
    Dk.merge_partials(o_p.view(rows, 1, D), lse_rows.view(rows, 1), H, 0,
                      inbox=(o_ptrs.data_ptr(), l_ptrs.data_ptr(), world, rank))
    symm_ring.barrier()
    io = inbox_o.local.view(torch.float32)
    il = inbox_l.local.view(torch.float32)
    out = torch.empty(B, ql, H, D, device=o_p.device, dtype=torch.bfloat16)
    lse_m = torch.empty(B, ql, H, device=o_p.device, dtype=torch.float32)
    Dk.merge_partials(io[slot * n_o:(slot + 1) * n_o].view(rows, world, D),
                      il[slot * n_l:(slot + 1) * n_l].view(rows, world), H, 0, out=out, lse_out=lse_m)
    return out, lse_m.permute(0, 2, 1).contiguous()


class RingInferenceAttention(torch.autograd.Function):
    """Differentiable fused path of ``ringattention_inference`` (gradients to q, k, v only,
    ringattention_inference.py:64)."""

    @staticmethod
    def forward(ctx, q, k, v, mask_local, axis, symm_ring):
        B, ql, H, D = q.shape
        ms = MaskSpec(causal_block_size=0, q_pos=Positions(0), k_pos=Positions(0))
        if mask_local is not None:
            ms.keep_q, ms.keep_k = flash.pack_mask(mask_local)
        if axis.size == 1:
            out, lse = flash.flash_fwd(q, k, v, ms)
        else:
            if symm_ring is None:
                raise RuntimeError("multi-rank inference attention needs a symmetric-memory ring")
            o_p, lse_p = flash.flash_fwd(q, k, v, ms, out_fp32=True)
            out, lse = _exchange_and_merge(o_p, lse_p, axis, symm_ring)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.ms, ctx.axis = ms, axis
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        B, ql, H, D = q.shape
        if dout.stride(3) != 1 or any(s % 8 for s in dout.stride()[:3]):
            dout = dout.contiguous()
        lse2, delta = flash.flash_bwd_prep(out, dout, lse)
        dq_acc = torch.zeros(B, ql, H, D, device=q.device, dtype=torch.float32)
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        flash.flash_bwd(q, k, v, dout, lse2, delta, ctx.ms, dq_acc, dk, dv, flash.DKV_STORE_BF16)
        if ctx.axis.size > 1:
            # dQ of the replicated queries is the sum of the per-shard contributions (a few MB at most)
            dist.all_reduce(dq_acc, group=ctx.axis.group)
        dq = torch.empty_like(q)
        K.cast_f32_to_bf16(dq_acc.view(B * ql, H * D), dq.view(B * ql, H * D))
        return dq, dk, dv, None, None, None


def ring_inference_attention(q, k, v, attn_mask, axis, symm_ring=None):
    """Dispatch of the fused inference op: the split-KV decode kernel for at most 8 query rows when no
    gradient is needed, the flash kernels otherwise."""
    B, ql, H, D = q.shape
    need_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if ql <= 8 and not need_grad:
        return Dk.ring_decode_attention(q, k, v, attn_mask, axis, symm_ring)
    S_loc = k.shape[1]
    m = _local_mask(attn_mask, axis.rank, S_loc, B, H, ql)

    def ok(t):
        return t.stride(3) == 1 and not any(s % 8 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0

    qq, kk, vv = (t if ok(t) else t.contiguous() for t in (q, k, v))
    return RingInferenceAttention.apply(qq, kk, vv, m, axis, symm_ring)
