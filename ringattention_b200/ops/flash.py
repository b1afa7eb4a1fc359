"""Low-level Python entry points of the sm_100a attention kernels (one ring step each).

``flash_fwd`` runs ``attn_fwd_sm100.cu``: local queries against one KV block with optional carry-in
``(o_prev, lse_prev)``, masks driven by global positions, and an optional in-kernel copy job that
pulls the *next* ring step's KV block from a peer GPU. ``flash_bwd`` runs ``attn_bwd_sm100.cu``.
Both take ``(B, S, H, D)`` bf16 views with a contiguous last dim (``D`` in {64, 128}).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

c_ll = ctypes.c_longlong
c_vp = ctypes.c_void_p


@dataclass
class Positions:
    """Global positions of a shard: one run ``[off0, off0+n)`` or two runs of ``half`` tokens."""

    off0: int
    off1: int = 0
    half: int = 1 << 30

    @classmethod
    def from_segments(cls, segs) -> "Positions":
        if len(segs) == 1:
            return cls(segs[0][1], 0, 1 << 30)
        (_, g0, n0), (l1, g1, _) = segs
        assert l1 == n0
        return cls(g0, g1, n0)

    def tensor(self, n: int, device) -> torch.Tensor:
        i = torch.arange(n, device=device)
        return torch.where(i < self.half, self.off0 + i, self.off1 + (i - self.half))


@dataclass
class MaskSpec:
    """Everything the kernels need to know about masking for one (q shard, kv block) pair."""

    causal_block_size: int = 0            # 0 = not causal
    q_pos: Positions = None               # type: ignore[assignment]
    k_pos: Positions = None               # type: ignore[assignment]
    seg_q: Optional[torch.Tensor] = None  # (B, Sq) int32, ids of the local queries
    seg_k: Optional[torch.Tensor] = None  # (B, Sk) int32, ids of this KV block
    seg_q_mm: Optional[torch.Tensor] = None
    seg_k_mm: Optional[torch.Tensor] = None
    bias: Optional[torch.Tensor] = None   # (B, 1|H, Sk) fp32 key bias for this KV block
    seed: int = 0
    pdrop: float = 0.0
    keep_q: Optional[torch.Tensor] = None  # (B, 1|H, Sq, 4*ceil(Sk/128)) int32 bitmap by query row (forward)
    keep_k: Optional[torch.Tensor] = None  # (B, 1|H, Sk, 4*ceil(Sq/128)) int32 bitmap by kv row (backward)


def seg_tile_minmax(seg: torch.Tensor) -> torch.Tensor:
    """Per-128-token-tile ``{min, max}`` of segment ids: ``(B, ceil(S/128), 2)`` int32."""
    B, S = seg.shape
    nt = (S + 127) // 128
    pad = nt * 128 - S
    if pad:
        seg = torch.cat([seg, seg[:, -1:].expand(B, pad)], dim=1)
    t = seg.view(B, nt, 128)
    return torch.stack([t.amin(dim=2), t.amax(dim=2)], dim=2).to(torch.int32).contiguous()


class _FwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_vp), ("k", c_vp), ("v", c_vp),
        ("q_sb", c_ll), ("q_ss", c_ll), ("q_sh", c_ll),
        ("k_sb", c_ll), ("k_ss", c_ll), ("k_sh", c_ll),
        ("v_sb", c_ll), ("v_ss", c_ll), ("v_sh", c_ll),
        ("out", c_vp), ("o_sb", c_ll), ("o_ss", c_ll), ("o_sh", c_ll), ("out_fp32", ctypes.c_int),
        ("lse_out", c_vp),
        ("o_prev", c_vp), ("lse_prev", c_vp),
        ("B", ctypes.c_int), ("H", ctypes.c_int), ("Sq", ctypes.c_int), ("Sk", ctypes.c_int),
        ("D", ctypes.c_int),
        ("softmax_scale", ctypes.c_float),
        ("causal_block_size", ctypes.c_int),
        ("q_off0", ctypes.c_int), ("q_off1", ctypes.c_int), ("q_half", ctypes.c_int),
        ("k_off0", ctypes.c_int), ("k_off1", ctypes.c_int), ("k_half", ctypes.c_int),
        ("seg_q", c_vp), ("seg_k", c_vp), ("seg_q_mm", c_vp), ("seg_k_mm", c_vp),
        ("bias", c_vp), ("bias_sb", c_ll), ("bias_sh", c_ll),
        ("seed", ctypes.c_ulonglong), ("drop_threshold", ctypes.c_uint),
        ("keep", c_vp), ("keep_sb", c_ll), ("keep_sh", c_ll), ("keep_sr", c_ll),
        ("copy_src", c_vp), ("copy_dst", c_vp), ("copy_bytes", c_ll), ("copy_ctas", ctypes.c_int),
        ("status", c_vp),
        ("stream", c_vp),
    ]


def _check_bshd(t: torch.Tensor, name: str) -> None:
    if t.dim() != 4 or t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(3) != 1:
        raise ValueError(f"{name} must be a CUDA bf16 (B, S, H, D) view with contiguous D")
    if any(s % 8 for s in t.stride()[:3]) or t.data_ptr() % 16:
        raise ValueError(f"{name}: strides must be multiples of 8 elements and base 16-byte aligned")


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def pack_mask(mask: torch.Tensor, want_q: bool = True, want_k: bool = True):
    """Pack a boolean ``(B, 1|H, 1|Sq, Sk)`` mask (True = attend) into the two bitmaps the kernels read:
    by query row for the forward, by kv row for the backward (``MaskSpec.keep_q`` / ``keep_k``). A mask
    without query rows (a key-padding mask) must be expanded by the caller to the query length first."""
    assert mask.dim() == 4 and mask.is_cuda
    m = mask.to(torch.uint8)
    if m.stride(3) != 1:
        m = m.contiguous()
    B, Hm, Sq, Sk = m.shape
    Wk, Wq = 4 * ((Sk + 127) // 128), 4 * ((Sq + 127) // 128)
    by_q = torch.zeros(B, Hm, Sq, Wk, device=m.device, dtype=torch.int32) if want_q else None
    by_k = torch.zeros(B, Hm, Sk, Wq, device=m.device, dtype=torch.int32) if want_k else None
    _lib.call("ra_pack_mask", c_vp(m.data_ptr()), c_ll(m.stride(0)), c_ll(m.stride(1)), c_ll(m.stride(2)),
              c_vp(_ptr(by_q)), c_vp(_ptr(by_k)), B, Hm, Sq, Sk, _lib.stream_ptr())
    return by_q, by_k


def _fill_mask(a, mask: MaskSpec, H: int, by_k: bool = False):
    keep = mask.keep_k if by_k else mask.keep_q
    if (mask.keep_q is not None or mask.keep_k is not None) and keep is None:
        raise ValueError("the mask bitmap for this pass is missing (pack_mask builds both)")
    if keep is not None:
        assert keep.dtype == torch.int32 and keep.dim() == 4 and keep.is_contiguous()
        a.keep = keep.data_ptr()
        a.keep_sb = keep.stride(0)
        a.keep_sh = keep.stride(1) if keep.shape[1] == H else 0
        a.keep_sr = keep.stride(2)
    a.causal_block_size = int(mask.causal_block_size or 0)
    a.q_off0, a.q_off1, a.q_half = mask.q_pos.off0, mask.q_pos.off1, mask.q_pos.half
    a.k_off0, a.k_off1, a.k_half = mask.k_pos.off0, mask.k_pos.off1, mask.k_pos.half
    a.seg_q, a.seg_k = _ptr(mask.seg_q), _ptr(mask.seg_k)
    a.seg_q_mm, a.seg_k_mm = _ptr(mask.seg_q_mm), _ptr(mask.seg_k_mm)
    if mask.bias is not None:
        bias = mask.bias
        assert bias.dtype == torch.float32 and bias.dim() == 3 and bias.stride(2) == 1
        a.bias = bias.data_ptr()
        a.bias_sb = bias.stride(0)
        a.bias_sh = bias.stride(1) if bias.shape[1] == H else 0
    a.seed = int(mask.seed) & (2**64 - 1)
    if mask.pdrop > 0.0:
        a.drop_threshold = max(1, min(int(mask.pdrop * 4294967296.0), 0xFFFFFFFF))
    else:
        a.drop_threshold = 0


def flash_fwd(q, k, v, mask: MaskSpec, *, o_prev=None, lse_prev=None, out_fp32=False,
              out=None, lse_out=None, copy_src: int = 0, copy_dst: int = 0, copy_bytes: int = 0,
              copy_ctas: int = 8):
    """One ring step of the forward. Returns ``(out, lse)``; ``out`` is ``(B,Sq,H,D)`` fp32 or
    bf16, ``lse`` is ``(B,H,Sq)`` fp32 (natural log). ``o_prev`` must be fp32 contiguous."""
    _check_bshd(q, "q"); _check_bshd(k, "k"); _check_bshd(v, "v")
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    dev = q.device
    if out is None:
        out = torch.empty(B, Sq, H, D, device=dev, dtype=torch.float32 if out_fp32 else torch.bfloat16)
    if lse_out is None:
        lse_out = torch.empty(B, H, Sq, device=dev, dtype=torch.float32)
    if o_prev is not None:
        assert o_prev.dtype == torch.float32 and o_prev.is_contiguous() and lse_prev is not None
    a = _FwdArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.q_sb, a.q_ss, a.q_sh = q.stride(0), q.stride(1), q.stride(2)
    a.k_sb, a.k_ss, a.k_sh = k.stride(0), k.stride(1), k.stride(2)
    a.v_sb, a.v_ss, a.v_sh = v.stride(0), v.stride(1), v.stride(2)
    a.out = out.data_ptr()
    a.o_sb, a.o_ss, a.o_sh = out.stride(0), out.stride(1), out.stride(2)
    a.out_fp32 = 1 if out.dtype == torch.float32 else 0
    a.lse_out = lse_out.data_ptr()
    a.o_prev, a.lse_prev = _ptr(o_prev), _ptr(lse_prev)
    a.B, a.H, a.Sq, a.Sk, a.D = B, H, Sq, Sk, D
    a.softmax_scale = 1.0 / math.sqrt(D)
    _fill_mask(a, mask, H)
    a.copy_src, a.copy_dst, a.copy_bytes, a.copy_ctas = copy_src, copy_dst, copy_bytes, copy_ctas
    a.status = _lib.status_tensor(dev).data_ptr()
    a.stream = torch.cuda.current_stream().cuda_stream
    _lib.call("ra_attn_fwd", ctypes.byref(a))
    return out, lse_out


class _BwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_vp), ("k", c_vp), ("v", c_vp), ("d_o", c_vp),
        ("q_sb", c_ll), ("q_ss", c_ll), ("q_sh", c_ll),
        ("k_sb", c_ll), ("k_ss", c_ll), ("k_sh", c_ll),
        ("v_sb", c_ll), ("v_ss", c_ll), ("v_sh", c_ll),
        ("do_sb", c_ll), ("do_ss", c_ll), ("do_sh", c_ll),
        ("lse2", c_vp), ("delta", c_vp), ("Sq_pad", ctypes.c_int),
        ("dq_acc", c_vp),
        ("dk", c_vp), ("dv", c_vp), ("dkv_sb", c_ll), ("dkv_ss", c_ll), ("dkv_sh", c_ll),
        ("dkv_mode", ctypes.c_int),
        ("B", ctypes.c_int), ("H", ctypes.c_int), ("Sq", ctypes.c_int), ("Sk", ctypes.c_int),
        ("D", ctypes.c_int),
        ("softmax_scale", ctypes.c_float),
        ("causal_block_size", ctypes.c_int),
        ("q_off0", ctypes.c_int), ("q_off1", ctypes.c_int), ("q_half", ctypes.c_int),
        ("k_off0", ctypes.c_int), ("k_off1", ctypes.c_int), ("k_half", ctypes.c_int),
        ("seg_q", c_vp), ("seg_k", c_vp), ("seg_q_mm", c_vp), ("seg_k_mm", c_vp),
        ("bias", c_vp), ("bias_sb", c_ll), ("bias_sh", c_ll),
        ("seed", ctypes.c_ulonglong), ("drop_threshold", ctypes.c_uint),
        ("keep", c_vp), ("keep_sb", c_ll), ("keep_sh", c_ll), ("keep_sr", c_ll),
        ("copy_src", c_vp), ("copy_dst", c_vp), ("copy_bytes", c_ll), ("copy_ctas", ctypes.c_int),
        ("status", c_vp),
        ("stream", c_vp),
        ("trace", c_vp),
    ]


# Phase-timestamp buffers by device index: a backward launch on that device records into its buffer
# (utils.tracing.BackwardPhaseTrace installs and removes them); launches on other devices are not traced.
BWD_TRACE_BUFFERS: dict = {}

DKV_STORE_BF16 = 0
DKV_STORE_FP32 = 1
DKV_REDUCE_FP32 = 2


def flash_bwd_prep(out, dout, lse):
    """``delta = rowsum(dO*O)`` and ``lse*log2(e)`` in ``(B, H, Sq_pad)`` fp32 buffers (padded to a
    multiple of 128 queries; padding and fully masked rows get ``+inf`` / 0)."""
    _check_bshd(out, "out"); _check_bshd(dout, "dout")
    B, Sq, H, D = out.shape
    sq_pad = (Sq + 127) // 128 * 128
    lse2 = torch.empty(B, H, sq_pad, device=out.device, dtype=torch.float32)
    delta = torch.empty(B, H, sq_pad, device=out.device, dtype=torch.float32)
    assert lse.dtype == torch.float32 and lse.is_contiguous() and lse.shape == (B, H, Sq)
    _lib.call("ra_attn_bwd_prep", c_vp(out.data_ptr()), c_ll(out.stride(0)), c_ll(out.stride(1)),
              c_ll(out.stride(2)), c_vp(dout.data_ptr()), c_ll(dout.stride(0)), c_ll(dout.stride(1)),
              c_ll(dout.stride(2)), c_vp(lse.data_ptr()), c_vp(lse2.data_ptr()),
              c_vp(delta.data_ptr()), B, H, Sq, sq_pad, D, _lib.stream_ptr())
    return lse2, delta


def flash_bwd(q, k, v, dout, lse2, delta, mask: MaskSpec, dq_acc, dk, dv, dkv_mode=DKV_STORE_BF16,
              *, copy_src: int = 0, copy_dst: int = 0, copy_bytes: int = 0, copy_ctas: int = 8):
    """One ring step of the backward. ``dq_acc`` (fp32, contiguous, pre-zeroed by the caller before
    the first step) receives ``dQ`` by reduction; ``dk``/``dv`` are written according to
    ``dkv_mode`` (store bf16, store fp32, or fp32 reduction into possibly remote memory)."""
    _check_bshd(q, "q"); _check_bshd(k, "k"); _check_bshd(v, "v"); _check_bshd(dout, "dout")
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    dev = q.device
    assert dq_acc.dtype == torch.float32 and dq_acc.is_contiguous() and dq_acc.shape == q.shape
    assert dk.shape == k.shape and dv.shape == k.shape and dk.stride() == dv.stride()
    want = torch.bfloat16 if dkv_mode == DKV_STORE_BF16 else torch.float32
    assert dk.dtype == want and dv.dtype == want and dk.stride(3) == 1
    a = _BwdArgs()
    a.q, a.k, a.v, a.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr()
    a.q_sb, a.q_ss, a.q_sh = q.stride(0), q.stride(1), q.stride(2)
    a.k_sb, a.k_ss, a.k_sh = k.stride(0), k.stride(1), k.stride(2)
    a.v_sb, a.v_ss, a.v_sh = v.stride(0), v.stride(1), v.stride(2)
    a.do_sb, a.do_ss, a.do_sh = dout.stride(0), dout.stride(1), dout.stride(2)
    a.lse2, a.delta, a.Sq_pad = lse2.data_ptr(), delta.data_ptr(), lse2.shape[2]
    a.dq_acc = dq_acc.data_ptr()
    a.dk, a.dv = dk.data_ptr(), dv.data_ptr()
    a.dkv_sb, a.dkv_ss, a.dkv_sh = dk.stride(0), dk.stride(1), dk.stride(2)
    a.dkv_mode = dkv_mode
    a.B, a.H, a.Sq, a.Sk, a.D = B, H, Sq, Sk, D
    a.softmax_scale = 1.0 / math.sqrt(D)
    _fill_mask(a, mask, H, by_k=True)
    a.copy_src, a.copy_dst, a.copy_bytes, a.copy_ctas = copy_src, copy_dst, copy_bytes, copy_ctas
    a.status = _lib.status_tensor(dev).data_ptr()
    a.stream = torch.cuda.current_stream().cuda_stream
    tb = BWD_TRACE_BUFFERS.get(dev.index if dev.index is not None else torch.cuda.current_device())
    a.trace = 0 if tb is None else tb.data_ptr()
    _lib.call("ra_attn_bwd", ctypes.byref(a))
