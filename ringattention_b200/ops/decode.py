"""Decode attention with a stationary, sequence-sharded KV cache (``decode_sm100.cu``).

``ring_decode_attention`` is the fused path of ``ringattention_inference``
(ringattention/ringattention_inference.py:8-35 rotates the whole cache; here only ``(o, lse)``
partials of ``B*H*q_len*(D+1)`` floats per rank cross NVLink, by stores into the peers' inboxes).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional

import torch

from . import _lib

c_ll = ctypes.c_longlong
c_vp = ctypes.c_void_p


# Depth of the split-KV kernel's asynchronous-copy ring for the cache rows (0: plain loads into registers).
# Measured on a 128K-row, 32-head shard: 5.25 TB/s with 0, 6.83 with 3, 6.84 with 4 (more shared memory per CTA).
STAGES = int(os.environ.get("RINGATTN_B200_DECODE_STAGES", "3"))


# Calls with at least this many query rows per cache row go to the tensor-core form of the split-KV kernel (the
# CUDA-core form spends q times the instructions per cache row).
MMA_MIN_ROWS = int(os.environ.get("RINGATTN_B200_DECODE_MMA_MIN_ROWS", "2"))


class _DecodeArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_vp), ("k", c_vp), ("v", c_vp),
        ("k_sb", c_ll), ("k_ss", c_ll), ("k_sh", c_ll), ("v_sb", c_ll), ("v_ss", c_ll), ("v_sh", c_ll),
        ("o_part", c_vp), ("lse_part", c_vp),
        ("mask", c_vp), ("m_sb", c_ll), ("m_sh", c_ll), ("m_sq", c_ll),
        ("B", ctypes.c_int), ("H", ctypes.c_int), ("QL", ctypes.c_int), ("S", ctypes.c_int),
        ("D", ctypes.c_int), ("splits", ctypes.c_int),
        ("softmax_scale", ctypes.c_float),
        ("q_pos0", c_ll), ("k_pos0", c_ll),
        ("pos_ptr", c_vp),
        ("stripe_n", ctypes.c_int), ("stripe_rank", ctypes.c_int),
        ("stripe_base", c_ll), ("stripe_len0", c_ll),
        ("stream", c_vp),
        ("stages", ctypes.c_int),
        ("mma", ctypes.c_int),
    ]


def _pad_q(q: torch.Tensor):
    """Pad the query length to 1, 2, 4 or 8 rows (the kernel holds them in registers)."""
    ql = q.shape[1]
    if ql > 8:
        raise ValueError("decode attention handles at most 8 query rows per call; use the prefill path")
    tgt = 1 if ql == 1 else (2 if ql == 2 else (4 if ql <= 4 else 8))
    if tgt != ql:
        pad = torch.zeros(q.shape[0], tgt - ql, q.shape[2], q.shape[3], device=q.device, dtype=q.dtype)
        q = torch.cat([q, pad], dim=1)
    return q.contiguous(), ql, tgt


def default_splits(S: int, B: int, H: int, mma: bool = False) -> int:
    """Many small CTAs: measured on a 128K-row, 32-head shard, 18 splits (4 CTAs per SM in total) gave
    4.57 TB/s, 74 splits 4.65 (a ragged last wave), 256 splits 5.19 with register loads; with the asynchronous-copy
    ring 64 to 512 splits are within 3 % of each other (6.83 to 7.02 TB/s). At least 512 cache rows per CTA.
    The tensor-core kernel (``mma``) has two CTAs of four warps per SM and likes half as many, longer ranges: four
    query rows, 128 / 256 / 512 splits: 0.315 / 0.332 / 0.408 ms."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    per_sm, rows = (32, 1024) if mma else (64, 512)
    want = max(1, (per_sm * sms) // max(1, B * H))
    return max(1, min(want, (S + rows - 1) // rows, 512))


def decode_partial(q, k, v, *, n_valid: Optional[int] = None, q_pos0: int = -1, k_pos0: int = 0,
                   mask: Optional[torch.Tensor] = None, splits: Optional[int] = None, pos_ptr: int = 0,
                   stripe: Optional[tuple] = None):
    """Split-KV pass over this rank's cache rows ``[0, n_valid)``. Returns fp32 partials
    ``(o_part (B*H*QL, splits, D), lse_part (B*H*QL, splits), QL_padded)``."""
    B, QL, H, D = q.shape
    S = k.shape[1] if n_valid is None else int(n_valid)
    splits = splits or default_splits(S, B, H, mma=QL >= MMA_MIN_ROWS)
    rows = B * H * QL
    o_part = torch.empty(rows, splits, D, device=q.device, dtype=torch.float32)
    lse_part = torch.empty(rows, splits, device=q.device, dtype=torch.float32)
    a = _DecodeArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.k_sb, a.k_ss, a.k_sh = k.stride(0), k.stride(1), k.stride(2)
    a.v_sb, a.v_ss, a.v_sh = v.stride(0), v.stride(1), v.stride(2)
    a.o_part, a.lse_part = o_part.data_ptr(), lse_part.data_ptr()
    if mask is not None:
        assert mask.dtype == torch.uint8 and mask.dim() == 4 and mask.stride(3) == 1
        a.mask = mask.data_ptr()
        a.m_sb = mask.stride(0) if mask.shape[0] > 1 else 0
        a.m_sh = mask.stride(1) if mask.shape[1] > 1 else 0
        a.m_sq = mask.stride(2) if mask.shape[2] > 1 else 0
    a.B, a.H, a.QL, a.S, a.D, a.splits = B, H, QL, S, D, splits
    a.softmax_scale = 1.0 / math.sqrt(D)
    a.q_pos0, a.k_pos0 = int(q_pos0), int(k_pos0)
    a.pos_ptr = pos_ptr
    # striped cache (with pos_ptr): (ranks, rank, prefilled rows per rank, prefilled positions)
    a.stripe_n, a.stripe_rank, a.stripe_base, a.stripe_len0 = stripe if stripe is not None else (0, 0, 0, 0)
    a.stream = torch.cuda.current_stream().cuda_stream
    a.stages = STAGES
    a.mma = int(QL >= MMA_MIN_ROWS)
    _lib.call("ra_decode_splitkv", ctypes.byref(a))
    return o_part, lse_part


def merge_partials(o_part, lse_part, H: int, QL: int, *, out=None, lse_out=None, inbox=None,
                   step_ptr: int = 0, slot_mul: int = 1, slot_add: int = 0, out_slot=(0, 0), in_slot=(0, 0)):
    """Merge ``nparts`` partials per row; ``o_part (rows, nparts, D)`` and ``lse_part (rows, nparts)``
    may be strided views. ``QL = 0`` writes rows in their own order (prefill); ``QL > 0`` maps row
    ``(b, h, i)`` to ``out[b, i, h]`` (decode). ``inbox = (o_ptrs, lse_ptrs, n_ranks, my_rank)`` makes the
    kernel also store the merged row into slot ``my_rank`` of every rank's inbox."""
    rows, nparts, D = o_part.shape
    assert o_part.stride(2) == 1
    o_ptrs = lse_ptrs = 0
    n_ranks = my_rank = 0
    if inbox is not None:
        o_ptrs, lse_ptrs, n_ranks, my_rank = inbox
    _lib.call("ra_decode_merge", c_vp(o_part.data_ptr()), c_vp(lse_part.data_ptr()),
              c_ll(o_part.stride(0)), c_ll(o_part.stride(1)), c_ll(lse_part.stride(0)),
              c_ll(lse_part.stride(1)), rows, nparts, D, H, QL,
              c_vp(0 if out is None else out.data_ptr()),
              0 if out is None else int(out.dtype == torch.float32),
              c_vp(0 if lse_out is None else lse_out.data_ptr()), c_vp(o_ptrs), c_vp(lse_ptrs),
              n_ranks, my_rank, c_vp(step_ptr), c_ll(slot_mul), c_ll(slot_add), c_ll(out_slot[0]), c_ll(out_slot[1]), c_ll(in_slot[0]),
              c_ll(in_slot[1]), _lib.stream_ptr())
    return out


def exchange_fits(rows: int) -> bool:
    """Whether the one-launch cross-GPU merge takes this many (batch, head, query) rows: all its CTAs have to be
    resident while they wait for their peers."""
    return rows <= _lib.lib().ra_decode_exchange_max_rows()


def merge_exchange(o_part, lse_part, H: int, QL: int, out, symm_ring) -> None:
    """Merge the split partials of every row, exchange the result with the other ranks of ``symm_ring`` by peer
    stores, wait per row for theirs and merge those into ``out``: one launch (no separate barrier, no second merge
    kernel). Collective over the ring; every rank must call it with the same shapes in the same order."""
    rows, nparts, D = o_part.shape
    world, rank = symm_ring.size, symm_ring.rank
    assert o_part.stride(2) == 1 and exchange_fits(rows)
    max_rows = _lib.lib().ra_decode_exchange_max_rows()
    box_o = symm_ring.buffer("decode_xchg_o", 2 * max_rows * world * D * 4)
    box_l = symm_ring.buffer("decode_xchg_lse", 2 * max_rows * world * 4)
    flags = symm_ring.buffer("decode_xchg_flags", max_rows * world * 4)
    sync = symm_ring.scratch_zeros("decode_xchg_sync", 8)
    _lib.call("ra_decode_merge_exchange", c_vp(o_part.data_ptr()), c_vp(lse_part.data_ptr()),
              c_ll(o_part.stride(0)), c_ll(o_part.stride(1)), c_ll(lse_part.stride(0)), c_ll(lse_part.stride(1)),
              rows, nparts, D, H, QL, c_vp(out.data_ptr()), int(out.dtype == torch.float32),
              c_vp(symm_ring.peer_ptr_table("decode_xchg_o").data_ptr()),
              c_vp(symm_ring.peer_ptr_table("decode_xchg_lse").data_ptr()),
              c_vp(box_o.ptr), c_vp(box_l.ptr), max_rows,
              c_vp(symm_ring.peer_ptr_table("decode_xchg_flags").data_ptr()),
              c_vp(sync.data_ptr()), world, rank, ctypes.c_ulonglong(symm_ring.timeout_ns),
              c_vp(_lib.status_tensor(o_part.device).data_ptr()), _lib.stream_ptr())


def ring_decode_attention(q, k, v, attn_mask, axis, symm_ring=None, *, n_valid: Optional[int] = None,
                          q_pos0: int = -1, k_pos0: Optional[int] = None, state: Optional[torch.Tensor] = None,
                          exchange: int = 0, exchanges_per_step: int = 1, stripe: Optional[tuple] = None):
    """``q (B, q_len<=8, H, D)`` replicated; ``k, v (B, kv_len, H, D)`` local cache shard; boolean
    ``attn_mask`` broadcastable to ``(B, H, q_len, S_total)``, global on the last axis (True =
    attend). Returns ``(B, q_len, H, D)`` in ``v.dtype``, identical on every rank."""
    rank, world = axis.rank, axis.size
    B, ql, H, D = q.shape
    S_loc = k.shape[1]
    qp, ql, QL = _pad_q(q)
    mask_u8 = None
    if attn_mask is not None:
        m = attn_mask
        while m.dim() < 4:
            m = m.unsqueeze(0)
        m = m[..., rank * S_loc:(rank + 1) * S_loc]
        if m.shape[2] not in (1, QL):
            pad = torch.zeros(*m.shape[:2], QL - m.shape[2], m.shape[3], dtype=m.dtype, device=m.device)
            m = torch.cat([m, pad], dim=2)
        mask_u8 = m.to(torch.uint8).contiguous()
    if k_pos0 is None:
        k_pos0 = rank * S_loc
    pos_ptr = 0 if state is None else state.data_ptr()
    step_ptr = 0 if state is None else state.data_ptr() + 8
    o_part, lse_part = decode_partial(qp, k, v, n_valid=n_valid, q_pos0=q_pos0, k_pos0=k_pos0, mask=mask_u8,
                                      pos_ptr=pos_ptr, stripe=stripe)
    out = torch.empty(B, QL, H, D, device=q.device, dtype=v.dtype)
    if world == 1:
        merge_partials(o_part, lse_part, H, QL, out=out)
        return out[:, :ql]
    if symm_ring is None:
        raise RuntimeError("multi-rank decode needs a symmetric-memory ring")
    rows = B * H * QL
    if exchange_fits(rows):
        merge_exchange(o_part, lse_part, H, QL, out, symm_ring)
        return out[:, :ql]
    # too many rows for the one-launch exchange: merge into the inboxes, barrier, merge the ranks
    inbox_o = symm_ring.buffer("decode_inbox_o", 2 * rows * world * D * 4)
    inbox_l = symm_ring.buffer("decode_inbox_lse", 2 * rows * world * 4)
    o_tab, l_tab = symm_ring.peer_ptr_table("decode_inbox_o"), symm_ring.peer_ptr_table("decode_inbox_lse")
    n_o, n_l = rows * world * D, rows * world  # floats per inbox slot
    io = inbox_o.local.view(torch.float32)
    il = inbox_l.local.view(torch.float32)
    if state is None:
        # double-buffered across calls (one barrier per call is enough); slot chosen on the host
        slot = symm_ring.calls & 1
        symm_ring.calls += 1
        o_ptrs = o_tab + slot * n_o * 4
        l_ptrs = l_tab + slot * n_l * 4
        merge_partials(o_part, lse_part, H, QL, inbox=(o_ptrs.data_ptr(), l_ptrs.data_ptr(), world, rank))
        symm_ring.barrier()
        merge_partials(io[slot * n_o:(slot + 1) * n_o].view(rows, world, D),
                       il[slot * n_l:(slot + 1) * n_l].view(rows, world), H, QL, out=out)
    else:
        # slot = (step * exchanges_per_step + exchange) & 1, from the device-side step counter
        sk = dict(step_ptr=step_ptr, slot_mul=exchanges_per_step, slot_add=exchange)
        merge_partials(o_part, lse_part, H, QL, inbox=(o_tab.data_ptr(), l_tab.data_ptr(), world, rank),
                       out_slot=(n_o, n_l), **sk)
        symm_ring.barrier()
        merge_partials(io[:n_o].view(rows, world, D), il[:n_l].view(rows, world), H, QL, out=out,
                       in_slot=(n_o, n_l), **sk)
    return out[:, :ql]


def shared_prefix_decode_attention(q, k_prefix, v_prefix, n_prefix: int, k_tail, v_tail, axis, symm_ring=None, *,
                                   state: torch.Tensor, stripe: tuple, exchange: int = 0, exchanges_per_step: int = 1,
                                   work: Optional[dict] = None):
    """Decode attention of ``S`` streams that share one cached prefix and have private tails.

    ``q (S, 1, H, D)``: one query per stream. ``k_prefix, v_prefix (1, rows, H, D)``: this rank's rows of the shared
    context, of which ``n_prefix`` are valid. ``k_tail, v_tail (S, T, H, D)``: this rank's rows of every stream's
    decoded tokens (striped over the ranks: ``stripe = (ranks, rank, 0, prefix positions)``; the number of valid
    rows comes from the position in ``state[0]`` on the device). The prefix is streamed once for all streams (the
    streams become the query rows of one split-KV call, at most 8), the tails are a second, tiny call; both are
    merged per stream with log-sum-exp weights and then across the ranks like any decode step. Returns ``(S, 1, H,
    D)`` in ``v``'s dtype, identical on every rank. ``work``: a dict that keeps the intermediate buffers between
    calls (needed under CUDA-graph capture, where addresses must not change)."""
    rank, world = axis.rank, axis.size
    S, one, H, D = q.shape
    assert one == 1 and S <= 8 and k_prefix.shape[0] == 1
    dev = q.device
    work = work if work is not None else {}
    rows = S * H
    if "o12" not in work:
        work["o12"] = torch.empty(2, rows, D, device=dev, dtype=torch.float32)
        work["l12"] = torch.empty(2, rows, device=dev, dtype=torch.float32)
    o12, l12 = work["o12"], work["l12"]
    # ---- shared prefix: the streams as query rows of one call (the cache is read once)
    qp, _, QL = _pad_q(q.view(1, S, H, D))
    o_p, lse_p = decode_partial(qp, k_prefix, v_prefix, n_valid=n_prefix, q_pos0=-1, k_pos0=0)
    if QL == S:
        merge_partials(o_p, lse_p, H, QL, out=o12[0].view(1, S, H, D), lse_out=l12[0])
    else:  # padded query rows: merge into a padded buffer, keep the first S
        if "pad_o" not in work:
            work["pad_o"] = torch.empty(1, QL, H, D, device=dev, dtype=torch.float32)
            work["pad_l"] = torch.empty(QL * H, device=dev, dtype=torch.float32)
        merge_partials(o_p, lse_p, H, QL, out=work["pad_o"], lse_out=work["pad_l"])
        o12[0].copy_(work["pad_o"][0, :S].reshape(rows, D))
        l12[0].copy_(work["pad_l"][:rows])
    # ---- private tails: one query per stream against its own rows on this rank
    o_t, lse_t = decode_partial(q.contiguous(), k_tail, v_tail, q_pos0=-1, k_pos0=0, pos_ptr=state.data_ptr(),
                                stripe=stripe, splits=1)
    merge_partials(o_t, lse_t, H, 1, out=o12[1].view(S, 1, H, D), lse_out=l12[1])
    # ---- the two partials of every (stream, head) row, then the ranks
    o_rows, l_rows = o12.permute(1, 0, 2), l12.permute(1, 0)            # (rows, 2, D), (rows, 2) views
    out = torch.empty(S, 1, H, D, device=dev, dtype=v_prefix.dtype)
    if world == 1:
        merge_partials(o_rows, l_rows, H, 0, out=out)
        return out
    if symm_ring is None:
        raise RuntimeError("multi-rank decode needs a symmetric-memory ring")
    if exchange_fits(rows):
        merge_exchange(o_rows, l_rows, H, 0, out, symm_ring)
        return out
    inbox_o = symm_ring.buffer("decode_inbox_o", 2 * rows * world * D * 4)
    inbox_l = symm_ring.buffer("decode_inbox_lse", 2 * rows * world * 4)
    o_tab, l_tab = symm_ring.peer_ptr_table("decode_inbox_o"), symm_ring.peer_ptr_table("decode_inbox_lse")
    n_o, n_l = rows * world * D, rows * world
    io, il = inbox_o.local.view(torch.float32), inbox_l.local.view(torch.float32)
    sk = dict(step_ptr=state.data_ptr() + 8, slot_mul=exchanges_per_step, slot_add=exchange)
    merge_partials(o_rows, l_rows, H, 0, inbox=(o_tab.data_ptr(), l_tab.data_ptr(), world, rank),
                   out_slot=(n_o, n_l), **sk)
    symm_ring.barrier()
    merge_partials(io[:n_o].view(rows, world, D), il[:n_l].view(rows, world), H, 0, out=out, in_slot=(n_o, n_l), **sk)
    return out
