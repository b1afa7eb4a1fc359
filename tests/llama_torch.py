"""Plain-PyTorch LLaMA forward on the same flat parameters: the oracle for the kernel-driven model
(loss-curve and gradient parity tests) and the CPU execution path. Uses autograd; no custom ops."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from ringattention_b200.config import LlamaConfig


def rope_torch(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """``x (B,S,H,D)``; rotate pairs ``(i, i + D/2)`` by ``pos * theta^(-2i/D)``."""
    D = x.shape[-1]
    i = torch.arange(D // 2, device=x.device, dtype=torch.float32)
    inv = torch.exp2(-math.log2(theta) * (2.0 * i / D))
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    cs, sn = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    a, c = x[..., : D // 2].float(), x[..., D // 2:].float()
    return torch.cat([a * cs - c * sn, c * cs + a * sn], dim=-1).to(x.dtype)


def rmsnorm_torch(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def llama_forward_torch(cfg: LlamaConfig, weights: dict, tokens: torch.Tensor,
                        targets: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
                        segment_ids: Optional[torch.Tensor] = None, compute_dtype=torch.bfloat16):
    """``weights`` maps the names of :class:`~ringattention_b200.models.llama.FlatParams` to
    tensors. Returns the sum of token losses when ``targets`` is given, else the logits. The
    rounding points mirror the kernel model (bf16 activations between ops, fp32 inside them)."""
    B, S = tokens.shape
    H, D, d = cfg.n_heads, cfg.head_dim, cfg.d_model
    pos = positions if positions is not None else torch.arange(S, device=tokens.device)
    cd = compute_dtype

    def lin(x, w):
        return (x.float() @ w.float().t()).to(cd)

    x = weights["embed"][tokens.long()].to(cd).view(B * S, d)
    cbs = cfg.causal_block_size
    qp = torch.div(pos, cbs, rounding_mode="floor")
    masked = qp[:, None] < qp[None, :]
    masked = masked[None, None]
    if segment_ids is not None:
        masked = masked | (segment_ids[:, :, None] != segment_ids[:, None, :])[:, None]
    for l in range(cfg.n_layers):
        h1 = rmsnorm_torch(x, weights[f"l{l}.n1"], cfg.rms_eps)
        qkv = lin(h1, weights[f"l{l}.wqkv"]).view(B, S, 3, H, D)
        q = rope_torch(qkv[:, :, 0], pos, cfg.rope_theta)
        k = rope_torch(qkv[:, :, 1], pos, cfg.rope_theta)
        v = qkv[:, :, 2]
        s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(D)
        s = s.masked_fill(masked, float("-inf"))
        p = torch.softmax(s, dim=-1)
        attn = torch.einsum("bhqk,bkhd->bqhd", p, v.float()).to(cd).reshape(B * S, d)
        x2 = (x.float() + attn.float() @ weights[f"l{l}.wo"].float().t()).to(cd)
        h2 = rmsnorm_torch(x2, weights[f"l{l}.n2"], cfg.rms_eps)
        gu = lin(h2, weights[f"l{l}.wgu"])
        Fd = cfg.d_ff
        a = (F.silu(gu[:, :Fd].float()) * gu[:, Fd:].float()).to(cd)
        x = (x2.float() + a.float() @ weights[f"l{l}.wd"].float().t()).to(cd)
    hf = rmsnorm_torch(x, weights["nf"], cfg.rms_eps)
    logits = lin(hf, weights["lm_head"])
    if targets is None:
        return logits.view(B, S, -1)
    t = targets.reshape(-1).long()
    valid = t >= 0
    loss = F.cross_entropy(logits.float()[valid], t[valid], reduction="sum")
    return loss
