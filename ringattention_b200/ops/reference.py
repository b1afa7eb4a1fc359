"""Pure-PyTorch restatement of the reference algorithm: oracle, CPU path and NCCL baseline.

Three layers, all device-agnostic:

* :func:`dense_attention` - an un-chunked softmax attention (fp64 by default) driven by explicit
  global token positions. It is the correctness oracle for everything else.
* :func:`blockwise_fwd` / :func:`blockwise_bwd` - the per-device chunked online-softmax update and
  its hand-written backward, the math of ringattention/ringattention_jax.py:99-270 (forward
  recurrence :138-144, five-GEMM backward :218-232, tile skipping :147-164).
* :class:`RingAttentionRef` - the ring layer (ringattention_jax.py:17-97): K/V rotate rank i ->
  i+1 through a :class:`~ringattention_b200.parallel.comm.RingComm`; in the backward dK/dV travel
  with their block and are home after N hops.

Deliberate differences from the reference (they remove numerical accidents, not features):
masks are boolean predicates and masked probabilities are exactly zero (the reference adds
``finfo.min`` and combines pieces with ``minimum``); a fully masked row yields zeros; softmax state is
always fp32; the tile-skip predicate is exact for every chunk size; the dropout mask is a
counter-based hash of ``(seed, b, h, q_pos, k_pos)`` so it is identical in forward and backward and
independent of the ring step; the forward ring does N-1 transfers.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from ..config import BlockwiseKwargs

_M32 = 0xFFFFFFFF


# --------------------------------------------------------------------------------------------
# positions / layouts
# --------------------------------------------------------------------------------------------
def layout_pairs(layout: str, world: int):
    """The half-chunk pair ``(a, b)`` of every rank for a two-run layout, or ``None`` for the contiguous one.

    The sequence is cut into ``2 * world`` half-chunks. ``"zigzag"`` gives rank r the half-chunks r and 2N-1-r
    (equal causal work on every rank). ``"pairs:a0-b0,a1-b1,..."`` names the pairing explicitly: any perfect
    matching of the half-chunks, e.g. one that balances the work of packed documents (``balanced_pairs``)."""
    if layout == "contiguous" or world == 1:
        return None
    if layout == "zigzag":
        return [(r, 2 * world - 1 - r) for r in range(world)]
    if layout.startswith("pairs:"):
        pairs = [tuple(int(x) for x in item.split("-")) for item in layout[len("pairs:"):].split(",")]
        if len(pairs) != world or sorted(c for pr in pairs for c in pr) != list(range(2 * world)):
            raise ValueError(f"layout {layout!r} is not a pairing of the {2 * world} half-chunks of {world} ranks")
        return pairs
    raise ValueError(f"unknown layout {layout!r}")


def balanced_pairs(segment_ids: torch.Tensor, world: int) -> str:
    """A ``"pairs:..."`` layout that balances the attention work of packed documents over the ring.

    ``segment_ids`` is ``(B, S)`` with ids that change at document boundaries (the rows a ring works on). Under a
    causal mask a token attends to the tokens of its own document up to itself, so the work of a half-chunk is
    the sum over its tokens of (position - start of its document + 1). Half-chunks are sorted by work and the
    heaviest is paired with the lightest, the second heaviest with the second lightest, and so on, which minimises
    the largest pair. Without document boundaries the work grows with the position and the result is the zig-zag
    pairing."""
    B, S = segment_ids.shape
    n = 2 * world
    if S % n:
        raise ValueError("sequence length must be divisible by 2 * ring size")
    seg = segment_ids.to(torch.int64)
    pos = torch.arange(S, device=seg.device).expand(B, S)
    is_start = torch.ones_like(seg, dtype=torch.bool)
    is_start[:, 1:] = seg[:, 1:] != seg[:, :-1]
    start = torch.cummax(torch.where(is_start, pos, torch.zeros_like(pos)), dim=1).values
    work = (pos - start + 1).double().view(B, n, S // n).sum(dim=(0, 2))
    order = torch.argsort(work, stable=True).tolist()
    pairs = [tuple(sorted((order[i], order[n - 1 - i]))) for i in range(world)]
    pairs.sort()
    return "pairs:" + ",".join(f"{a}-{b}" for a, b in pairs)


def shard_positions(rank: int, world: int, local_len: int, layout: str = "contiguous",
                    device=None) -> torch.Tensor:
    """Global token positions held by ``rank`` (int64, ``local_len`` entries)."""
    pairs = layout_pairs(layout, world)
    if pairs is None:
        return torch.arange(rank * local_len, (rank + 1) * local_len, device=device)
    if local_len % 2:
        raise ValueError("a two-run layout needs an even local length")
    h = local_len // 2
    a, b = pairs[rank]
    return torch.cat([torch.arange(a * h, (a + 1) * h, device=device), torch.arange(b * h, (b + 1) * h, device=device)])


def shard_segments(rank: int, world: int, local_len: int, layout: str = "contiguous"):
    """The shard as a list of ``(local_start, global_start, length)`` contiguous runs."""
    pairs = layout_pairs(layout, world)
    if pairs is None:
        return [(0, rank * local_len, local_len)]
    h = local_len // 2
    a, b = pairs[rank]
    return [(0, a * h, h), (h, b * h, h)]


def to_layout(x: torch.Tensor, world: int, layout: str, dim: int = 1) -> torch.Tensor:
    """Reorder a *global* sequence so that equal contiguous slices are the per-rank shards."""
    if layout == "contiguous" or world == 1:
        return x
    s = x.shape[dim]
    idx = torch.cat([shard_positions(r, world, s // world, layout, x.device) for r in range(world)])
    return x.index_select(dim, idx)


def from_layout(x: torch.Tensor, world: int, layout: str, dim: int = 1) -> torch.Tensor:
    """Inverse of :func:`to_layout`."""
    if layout == "contiguous" or world == 1:
        return x
    s = x.shape[dim]
    idx = torch.cat([shard_positions(r, world, s // world, layout, x.device) for r in range(world)])
    inv = torch.empty_like(idx)
    inv[idx] = torch.arange(s, device=x.device)
    return x.index_select(dim, inv)


# --------------------------------------------------------------------------------------------
# counter-based dropout
# --------------------------------------------------------------------------------------------
def _mix32(x: torch.Tensor) -> torch.Tensor:
    x = x & _M32
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & _M32
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & _M32
    x = x ^ (x >> 16)
    return x


def dropout_hash(seed: int, bh: torch.Tensor, q_pos: torch.Tensor, k_pos: torch.Tensor) -> torch.Tensor:
    """32-bit hash of ``(seed, batch*H+head, q_pos, k_pos)``; the CUDA kernels compute the same
    function, so a mask drawn here is bit-identical to the one a kernel applies."""
    s_lo = seed & _M32
    s_hi = (seed >> 32) & _M32
    x = (q_pos * 0x9E3779B1 + k_pos * 0x85EBCA77 + bh * 0xC2B2AE3D + s_lo) & _M32
    x = _mix32(x)
    x = _mix32((x ^ s_hi) + (k_pos & _M32))
    return x


def dropout_threshold(p: float) -> int:
    return min(int(p * 4294967296.0), _M32)


def dropped(seed: int, p: float, batch: int, heads: int, q_pos: torch.Tensor,
            k_pos: torch.Tensor) -> torch.Tensor:
    """Boolean ``(B, H, Sq, Sk)``: True where the logit is dropped."""
    dev = q_pos.device
    bh = (torch.arange(batch, device=dev)[:, None] * heads + torch.arange(heads, device=dev)[None, :])
    h = dropout_hash(seed, bh[:, :, None, None].long(), q_pos.long()[None, None, :, None],
                     k_pos.long()[None, None, None, :])
    return h < dropout_threshold(p)


# --------------------------------------------------------------------------------------------
# mask predicate (True = masked)
# --------------------------------------------------------------------------------------------
def masked_predicate(q_pos: torch.Tensor, k_pos: torch.Tensor, batch: int, heads: int,
                     causal_block_size: Optional[int], seg_q: Optional[torch.Tensor],
                     seg_k: Optional[torch.Tensor], seed: int = 0, pdrop: float = 0.0,
                     extra_masked: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Union of the causal, segment and dropout rules; broadcastable to ``(B, H, Sq, Sk)``.

    ``seg_q``/``seg_k`` are the segment ids of exactly these q/k tokens (``(B, Sq)``, ``(B, Sk)``).
    """
    m = None
    if causal_block_size is not None:
        cbs = int(causal_block_size)
        c = (torch.div(q_pos, cbs, rounding_mode="floor")[:, None]
             < torch.div(k_pos, cbs, rounding_mode="floor")[None, :])
        m = c[None, None]
    if seg_q is not None:
        s = (seg_q[:, :, None] != seg_k[:, None, :])[:, None]
        m = s if m is None else (m | s)
    if pdrop > 0.0:
        d = dropped(seed, pdrop, batch, heads, q_pos, k_pos)
        m = d if m is None else (m | d)
    if extra_masked is not None:
        m = extra_masked if m is None else (m | extra_masked)
    return m


def bias_slice(bias: Optional[torch.Tensor], q_pos: torch.Tensor, k_pos: torch.Tensor,
               q_local: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Additive bias for these tokens. ``bias`` is global along keys: ``(B, 1|H, R, S_total)`` with
    R = 1 (key bias, the form the reference handles exactly, ringattention_jax.py:278-283), R =
    S_total (rows indexed by global query position) or R = number of local queries."""
    if bias is None:
        return None
    b = bias.index_select(-1, k_pos)
    r = bias.shape[-2]
    if r == 1:
        return b
    if q_local is not None and r == q_local.numel():
        return b.index_select(-2, q_local)
    return b.index_select(-2, q_pos)


# --------------------------------------------------------------------------------------------
# dense oracle
# --------------------------------------------------------------------------------------------
def dense_attention(q, k, v, q_pos=None, k_pos=None, *, causal_block_size=None, bias=None,
                    seg_q=None, seg_k=None, seed=0, pdrop=0.0, extra_masked=None,
                    dtype=torch.float64, return_lse=False):
    """Softmax attention of ``q (B,Sq,H,D)`` against ``k,v (B,Sk,H,D)`` with explicit positions.

    ``bias`` must already be sliced to ``(B, 1|H, 1|Sq, Sk)``. Returns ``(B,Sq,H,D)`` in ``dtype``.
    """
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    dev = q.device
    if q_pos is None:
        q_pos = torch.arange(Sq, device=dev)
    if k_pos is None:
        k_pos = torch.arange(Sk, device=dev)
    qf, kf, vf = q.to(dtype), k.to(dtype), v.to(dtype)
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) / math.sqrt(D)
    if bias is not None:
        s = s + bias.to(dtype)
    m = masked_predicate(q_pos, k_pos, B, H, causal_block_size, seg_q, seg_k, seed, pdrop,
                         extra_masked)
    if m is not None:
        s = s.masked_fill(m, float("-inf"))
    mx = s.amax(dim=-1, keepdim=True)
    mx = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
    p = torch.exp(s - mx)
    l = p.sum(dim=-1, keepdim=True)
    out = torch.einsum("bhqk,bkhd->bqhd", p / torch.where(l > 0, l, torch.ones_like(l)), vf)
    if return_lse:
        lse = (mx + torch.log(l)).squeeze(-1)  # -inf for fully masked rows
        return out, lse
    return out


# --------------------------------------------------------------------------------------------
# blockwise (chunked) forward / backward with carry
# --------------------------------------------------------------------------------------------
def tile_visible(q_pos_tile: torch.Tensor, k_pos_tile: torch.Tensor, cbs: Optional[int]) -> bool:
    """False when the causal rule masks every entry of the tile (exact; the reference's
    ``below_or_on_diag``, ringattention_jax.py:324-331, is off by one for chunk size 1)."""
    if cbs is None:
        return True
    return int(q_pos_tile.max()) // cbs >= int(k_pos_tile.min()) // cbs


def new_carry(B, Sq, H, D, device, dtype=torch.float32):
    """(acc, l, m): un-normalised output, row sum, row max (ringattention_jax.py:22-23,49)."""
    return (torch.zeros(B, Sq, H, D, device=device, dtype=dtype),
            torch.zeros(B, H, Sq, device=device, dtype=dtype),
            torch.full((B, H, Sq), float("-inf"), device=device, dtype=dtype))


def blockwise_fwd(q, k, v, carry, q_pos, k_pos, kw: BlockwiseKwargs, *, bias=None, seg_q=None,
                  seg_k=None, seed=0, extra_masked=None, acc_dtype=torch.float32):
    """One ring step: fold the KV block ``k, v`` into ``carry`` chunk by chunk."""
    acc, l, m = carry
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    qc = min(kw.query_chunk_size, Sq)
    kc = min(kw.key_chunk_size, Sk)
    if Sq % qc or Sk % kc:
        raise ValueError(f"chunk sizes ({qc},{kc}) must divide the local lengths ({Sq},{Sk})")
    scale = 1.0 / math.sqrt(D)
    pdrop = float(kw.attn_pdrop) if kw.dropout_active else 0.0
    acc, l, m = acc.clone(), l.clone(), m.clone()
    for qi in range(0, Sq, qc):
        qs = slice(qi, qi + qc)
        qt = q[:, qs].to(acc_dtype)
        a_t, l_t, m_t = acc[:, qs], l[:, :, qs], m[:, :, qs]
        for ki in range(0, Sk, kc):
            ks = slice(ki, ki + kc)
            if not tile_visible(q_pos[qs], k_pos[ks], kw.causal_block_size):
                continue
            s = torch.einsum("bqhd,bkhd->bhqk", qt, k[:, ks].to(acc_dtype)) * scale
            if bias is not None:
                bt = bias[..., ks] if bias.shape[-2] == 1 else bias[..., qs, ks]
                s = s + bt.to(acc_dtype)
            msk = masked_predicate(
                q_pos[qs], k_pos[ks], B, H, kw.causal_block_size,
                None if seg_q is None else seg_q[:, qs], None if seg_k is None else seg_k[:, ks],
                seed, pdrop, None if extra_masked is None else extra_masked[..., qs, ks])
            if msk is not None:
                s = s.masked_fill(msk, float("-inf"))
            m_new = torch.maximum(m_t, s.amax(dim=-1))
            m_safe = torch.where(torch.isfinite(m_new), m_new, torch.zeros_like(m_new))
            p = torch.exp(s - m_safe[..., None])
            alpha = torch.exp(torch.where(torch.isfinite(m_t), m_t - m_safe, torch.full_like(m_t, float("-inf"))))
            l_t = alpha * l_t + p.sum(dim=-1)
            a_t = a_t * alpha.permute(0, 2, 1)[..., None] + torch.einsum(
                "bhqk,bkhd->bqhd", p, v[:, ks].to(acc_dtype))
            m_t = m_new
        acc[:, qs], l[:, :, qs], m[:, :, qs] = a_t, l_t, m_t
    return acc, l, m


def finalize(carry, out_dtype):
    """``O = acc / l`` (zeros for fully masked rows) and ``lse = m + log l``."""
    acc, l, m = carry
    safe = torch.where(l > 0, l, torch.ones_like(l))
    out = acc / safe.permute(0, 2, 1)[..., None]
    lse = torch.where(l > 0, m + torch.log(safe), torch.full_like(m, float("-inf")))
    return out.to(out_dtype), lse


def blockwise_bwd(q, k, v, out, lse, dout, q_pos, k_pos, kw: BlockwiseKwargs, *, bias=None,
                  seg_q=None, seg_k=None, seed=0, extra_masked=None, acc_dtype=torch.float32):
    """Gradients of one (local q, KV block) pair given the *final* ``out`` and ``lse``.

    Returns ``(dq, dk, dv)`` in ``acc_dtype``: ``P = exp(S - lse)``, ``dV = P^T dO``,
    ``dP = dO V^T``, ``dS = P * (dP - rowsum(dO*O))``, ``dQ = dS K / sqrt(D)``,
    ``dK = dS^T Q / sqrt(D)`` (ringattention_jax.py:218-232).
    """
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    qc = min(kw.query_chunk_size, Sq)
    kc = min(kw.key_chunk_size, Sk)
    scale = 1.0 / math.sqrt(D)
    pdrop = float(kw.attn_pdrop) if kw.dropout_active else 0.0
    dq = torch.zeros(B, Sq, H, D, device=q.device, dtype=acc_dtype)
    dk = torch.zeros(B, Sk, H, D, device=q.device, dtype=acc_dtype)
    dv = torch.zeros(B, Sk, H, D, device=q.device, dtype=acc_dtype)
    delta = torch.einsum("bqhd,bqhd->bhq", dout.to(acc_dtype), out.to(acc_dtype))
    for qi in range(0, Sq, qc):
        qs = slice(qi, qi + qc)
        qt = q[:, qs].to(acc_dtype)
        dot = dout[:, qs].to(acc_dtype)
        lse_t = lse[:, :, qs].to(acc_dtype)
        lse_safe = torch.where(torch.isfinite(lse_t), lse_t, torch.zeros_like(lse_t))
        for ki in range(0, Sk, kc):
            ks = slice(ki, ki + kc)
            if not tile_visible(q_pos[qs], k_pos[ks], kw.causal_block_size):
                continue
            kt, vt = k[:, ks].to(acc_dtype), v[:, ks].to(acc_dtype)
            s = torch.einsum("bqhd,bkhd->bhqk", qt, kt) * scale
            if bias is not None:
                bt = bias[..., ks] if bias.shape[-2] == 1 else bias[..., qs, ks]
                s = s + bt.to(acc_dtype)
            msk = masked_predicate(
                q_pos[qs], k_pos[ks], B, H, kw.causal_block_size,
                None if seg_q is None else seg_q[:, qs], None if seg_k is None else seg_k[:, ks],
                seed, pdrop, None if extra_masked is None else extra_masked[..., qs, ks])
            if msk is not None:
                s = s.masked_fill(msk, float("-inf"))
            p = torch.exp(s - lse_safe[..., None])
            p = torch.where(torch.isfinite(lse_t)[..., None], p, torch.zeros_like(p))
            dv[:, ks] += torch.einsum("bhqk,bqhd->bkhd", p, dot)
            dp = torch.einsum("bqhd,bkhd->bhqk", dot, vt)
            ds = p * (dp - delta[:, :, qs, None])
            dq[:, qs] += torch.einsum("bhqk,bkhd->bqhd", ds, kt) * scale
            dk[:, ks] += torch.einsum("bhqk,bqhd->bkhd", ds, qt) * scale
    return dq, dk, dv


def merge_partials(o_a, lse_a, o_b, lse_b):
    """Merge two normalised partial results: ``lse = logaddexp``; outputs are re-weighted.
    ``o`` is ``(B,S,H,D)``, ``lse`` is ``(B,H,S)``. Rows with ``lse = -inf`` on both sides stay zero."""
    lse = torch.logaddexp(lse_a, lse_b)
    safe = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse))
    wa = torch.exp(lse_a - safe).permute(0, 2, 1)[..., None]
    wb = torch.exp(lse_b - safe).permute(0, 2, 1)[..., None]
    wa = torch.nan_to_num(wa, nan=0.0)
    wb = torch.nan_to_num(wb, nan=0.0)
    return o_a * wa + o_b * wb, lse


# --------------------------------------------------------------------------------------------
# ring layer over a RingComm
# --------------------------------------------------------------------------------------------
def _ring_positions(comm, Sq, Sk, cache_idx, layout, device):
    rank, world = comm.rank, comm.size
    if cache_idx is None:
        q_pos = shard_positions(rank, world, Sq, layout, device)
    else:  # q is replicated and starts at cache_idx on every rank (ringattention_jax.py:34-35)
        q_pos = torch.arange(int(cache_idx), int(cache_idx) + Sq, device=device)
    return q_pos, (lambda j: shard_positions(j, world, Sk, layout, device))


class RingAttentionRef(torch.autograd.Function):
    """Ring attention by rotation, the reference algorithm. Works on CPU (gloo / in-process fake
    ring) and on GPU with NCCL send/recv, where it serves as the baseline the fused path beats."""

    @staticmethod
    def forward(ctx, q, k, v, bias, segment_ids, cache_idx, comm, float32_logits, kw):
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        dev = q.device
        acc_dtype = torch.float64 if q.dtype == torch.float64 else torch.float32
        rank, world = comm.rank, comm.size
        seed = kw.seed()
        q_pos, k_pos_of = _ring_positions(comm, Sq, Sk, cache_idx, kw.layout, dev)
        seg_q = None if segment_ids is None else segment_ids.index_select(1, q_pos)
        carry = new_carry(B, Sq, H, D, dev, acc_dtype)
        kt, vt = k, v
        for t in range(world):
            j = (rank - t) % world
            k_pos = k_pos_of(j)
            seg_k = None if segment_ids is None else segment_ids.index_select(1, k_pos)
            carry = blockwise_fwd(q, kt, vt, carry, q_pos, k_pos, kw,
                                  bias=bias_slice(bias, q_pos, k_pos, torch.arange(Sq, device=dev)),
                                  seg_q=seg_q, seg_k=seg_k, seed=seed, acc_dtype=acc_dtype)
            if t + 1 < world:
                kt, vt = comm.send_recv([kt, vt])
        out, lse = finalize(carry, v.dtype)
        ctx.save_for_backward(q, k, v, out, lse, bias, segment_ids)
        ctx.misc = (cache_idx, comm, kw, seed, acc_dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, bias, segment_ids = ctx.saved_tensors
        cache_idx, comm, kw, seed, acc_dtype = ctx.misc
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        dev = q.device
        rank, world = comm.rank, comm.size
        q_pos, k_pos_of = _ring_positions(comm, Sq, Sk, cache_idx, kw.layout, dev)
        seg_q = None if segment_ids is None else segment_ids.index_select(1, q_pos)
        dq = torch.zeros(B, Sq, H, D, device=dev, dtype=acc_dtype)
        dk = torch.zeros(B, Sk, H, D, device=dev, dtype=acc_dtype)
        dv = torch.zeros(B, Sk, H, D, device=dev, dtype=acc_dtype)
        kt, vt = k, v
        dout = dout.contiguous()
        for t in range(world):
            j = (rank - t) % world
            k_pos = k_pos_of(j)
            seg_k = None if segment_ids is None else segment_ids.index_select(1, k_pos)
            dq_t, dk_t, dv_t = blockwise_bwd(
                q, kt, vt, out, lse, dout, q_pos, k_pos, kw,
                bias=bias_slice(bias, q_pos, k_pos, torch.arange(Sq, device=dev)),
                seg_q=seg_q, seg_k=seg_k, seed=seed, acc_dtype=acc_dtype)
            dq += dq_t
            dk += dk_t
            dv += dv_t
            # K, V, dK, dV travel together; after N hops dK/dV are home (ringattention_jax.py:85-88)
            if world > 1:
                kt, vt, dk, dv = comm.send_recv([kt, vt, dk, dv])
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None, None, None, None)


def ring_attention_ref(q, k, v, attn_bias=None, segment_ids=None, cache_idx=None, comm=None,
                       float32_logits=True, blockwise_kwargs=None):
    """Functional form of :class:`RingAttentionRef`."""
    from ..parallel.comm import SingleComm

    kw = BlockwiseKwargs.from_any(blockwise_kwargs)
    return RingAttentionRef.apply(q, k, v, attn_bias, segment_ids, cache_idx,
                                  comm if comm is not None else SingleComm(), float32_logits, kw)


class RingAttentionInferenceRef(torch.autograd.Function):
    """Un-chunked ring attention with a boolean ``attn_mask`` that is global along keys, the
    algorithm of ringattention/ringattention_inference.py:8-64 (the whole KV shard rotates)."""

    @staticmethod
    def forward(ctx, q, k, v, attn_mask, comm, float32_logits):
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        dev = q.device
        rank, world = comm.rank, comm.size
        acc_dtype = torch.float64 if q.dtype == torch.float64 else torch.float32
        kw = BlockwiseKwargs(query_chunk_size=Sq, key_chunk_size=Sk)
        carry = new_carry(B, Sq, H, D, dev, acc_dtype)
        q_pos = torch.zeros(Sq, dtype=torch.long, device=dev)
        kt, vt = k, v
        for t in range(world):
            j = (rank - t) % world
            k_pos = torch.arange(j * Sk, (j + 1) * Sk, device=dev)
            extra = None if attn_mask is None else ~attn_mask[..., j * Sk:(j + 1) * Sk]
            carry = blockwise_fwd(q, kt, vt, carry, q_pos, k_pos, kw, extra_masked=extra,
                                  acc_dtype=acc_dtype)
            if t + 1 < world:
                kt, vt = comm.send_recv([kt, vt])
        out, lse = finalize(carry, v.dtype)
        ctx.save_for_backward(q, k, v, out, lse, attn_mask)
        ctx.misc = (comm, kw, acc_dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, attn_mask = ctx.saved_tensors
        comm, kw, acc_dtype = ctx.misc
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        dev = q.device
        rank, world = comm.rank, comm.size
        q_pos = torch.zeros(Sq, dtype=torch.long, device=dev)
        dq = torch.zeros(B, Sq, H, D, device=dev, dtype=acc_dtype)
        dk = torch.zeros(B, Sk, H, D, device=dev, dtype=acc_dtype)
        dv = torch.zeros(B, Sk, H, D, device=dev, dtype=acc_dtype)
        kt, vt = k, v
        for t in range(world):
            j = (rank - t) % world
            k_pos = torch.arange(j * Sk, (j + 1) * Sk, device=dev)
            extra = None if attn_mask is None else ~attn_mask[..., j * Sk:(j + 1) * Sk]
            dq_t, dk_t, dv_t = blockwise_bwd(q, kt, vt, out, lse, dout, q_pos, k_pos, kw,
                                             extra_masked=extra, acc_dtype=acc_dtype)
            dq += dq_t
            dk += dk_t
            dv += dv_t
            if world > 1:
                kt, vt, dk, dv = comm.send_recv([kt, vt, dk, dv])
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None, None
