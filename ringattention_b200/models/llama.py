"""LLaMA-style decoder driven by the sm_100a kernels, with hand-written forward and backward.

The reference has no model; its README shows the op inside an external LLaMA (LWM) on a
``(dp, fsdp, tp, sp)`` mesh (README.md:19-49,62). This driver supplies that model: RMSNorm, fused
QKV projection, RoPE, ring attention, output projection with the residual add in the GEMM epilogue,
blockwise SwiGLU feed-forward (chunk loop, ringattention_jax.py:333-352), chunked LM head fused with
the loss. Parameters live in flat buffers (fp32 master + moments + grads, bf16 working copy) so the
optimizer, the gradient all-reduce and checkpoints are single operations.

Remat policy ``nothing_saveable`` (ringattention_jax.py:334) keeps only the layer inputs and
recomputes each layer, attention included, in the backward pass. ``everything_saveable`` keeps the
per-layer activations that backward needs. ``save_attention`` (an extension) recomputes the layer
but keeps the attention output and log-sum-exp, so the ring forward runs once per layer and step.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..config import POLICY_NOTHING_SAVEABLE, POLICY_SAVE_ATTENTION, BlockwiseKwargs, LlamaConfig
from ..ops import attention as A
from ..ops import ffn
from ..ops import kernels as K
from ..ops.flash import Positions
from ..ops.reference import shard_segments
from ..utils.tracing import phase
from .params import FlatParams


@dataclass
class StepContext:
    """Per-step sharding information shared by all layers."""

    B: int
    S: int                      # local sequence length
    plan: A.RingPlan
    positions: Positions        # global positions of the local tokens (RoPE, masks)
    symm_ring: object = None
    total_tokens: int = 0       # number of target tokens in the whole global batch


class _LayerFFNLinears:
    """The feed-forward products of layer ``l`` on the flat (optionally fsdp-sharded) parameters, in the form
    ``ops.ffn.ffn_forward`` / ``ffn_backward`` call them."""

    def __init__(self, P: FlatParams, l: int):
        self.P, self.gu, self.d = P, f"l{l}.wgu", f"l{l}.wd"

    def gate_up(self, x):
        return self.P.lin_fwd(x, self.gu)

    def gate_up_act(self, x):
        if self.P.shard_count == 1:
            with phase("linear"):
                return K.linear_swiglu(x, self.P.w(self.gu))
        return K.swiglu_fwd(self.P.lin_fwd(x, self.gu))  # rows gathered inside the GEMM: activation apart

    def down(self, a, out, residual):
        return self.P.lin_fwd(a, self.d, out=out, residual=residual)

    def down_dgrad(self, dy):
        return self.P.lin_dgrad(dy, self.d)

    def down_wgrad(self, dy, a):
        self.P.lin_wgrad(dy, a, self.d)

    def gate_up_wgrad(self, dgu, x):
        self.P.lin_wgrad(dgu, x, self.gu)

    def gate_up_dgrad(self, dgu, out):
        return self.P.lin_dgrad(dgu, self.gu, out=out)


class LlamaModel:
    """Forward/backward of the decoder on one rank's token shard."""

    def __init__(self, cfg: LlamaConfig, device="cuda", seed: int = 0, with_optimizer: bool = True,
                 params: Optional[FlatParams] = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.params = params if params is not None else FlatParams(cfg, self.device, seed, with_optimizer)
        self.H, self.D = cfg.n_heads, cfg.head_dim
        if self.D not in (64, 128):
            raise ValueError("head_dim must be 64 or 128 for the fused attention kernels")

    # ------------------------------------------------------------------ context
    def make_context(self, B: int, S_local: int, rank: int = 0, world: int = 1, segment_ids=None,
                     symm_ring=None, total_tokens: Optional[int] = None, layout: Optional[str] = None) -> StepContext:
        """``layout`` overrides the configured token layout for this context (the trainer passes the pairing that
        balances a packed batch)."""
        layout = layout or self.cfg.layout
        kw = BlockwiseKwargs(causal_block_size=self.cfg.causal_block_size,
                             query_chunk_size=min(self.cfg.query_chunk_size, S_local),
                             key_chunk_size=min(self.cfg.key_chunk_size, S_local),
                             layout=layout)
        plan = A.make_plan(rank, world, B, S_local, S_local, self.H, kw, segment_ids=segment_ids,
                           device=self.device)
        pos = Positions.from_segments(shard_segments(rank, world, S_local, layout))
        return StepContext(B=B, S=S_local, plan=plan, positions=pos, symm_ring=symm_ring,
                           total_tokens=total_tokens if total_tokens is not None else B * S_local * world)

    # ------------------------------------------------------------------ layer forward
    def _attn_block_fwd(self, l: int, x: torch.Tensor, ctx: StepContext, kept_attn=None):
        """``kept_attn = (attn, lse)`` from the forward pass skips the ring forward (recomputation under
        the ``save_attention`` policy)."""
        cfg, P = self.cfg, self.params
        B, S, H, D, d = ctx.B, ctx.S, self.H, self.D, cfg.d_model
        h1, rstd1 = K.rmsnorm_fwd(x, P.w(f"l{l}.n1"), cfg.rms_eps)
        qkv = P.lin_fwd(h1, f"l{l}.wqkv")
        qkv5 = qkv.view(B, S, 3, H, D)
        qk = qkv.view(B, S, 3 * H, D)[:, :, :2 * H]  # q heads then k heads
        K.rope_(qk, ctx.positions, cfg.rope_theta)
        q, k, v = qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2]
        if kept_attn is not None:
            attn, lse = kept_attn
        else:
            with phase("attn_fwd"):
                attn, lse = A.ring_forward(q, k, v, ctx.plan, ctx.symm_ring)
        x2 = P.lin_fwd(attn.view(B * S, d), f"l{l}.wo", residual=x)
        return x2, (h1, rstd1, qkv, attn, lse)

    def _ffn_fwd(self, l: int, x2: torch.Tensor, h2: torch.Tensor) -> torch.Tensor:
        return ffn.ffn_forward(_LayerFFNLinears(self.params, l), h2, self.cfg.ffn_chunk_size, residual=x2)

    def layer_forward(self, l: int, x: torch.Tensor, ctx: StepContext, keep: bool = False):
        x2, saved = self._attn_block_fwd(l, x, ctx)
        h2, rstd2 = K.rmsnorm_fwd(x2, self.params.w(f"l{l}.n2"), self.cfg.rms_eps)
        x3 = self._ffn_fwd(l, x2, h2)
        if keep:
            return x3, saved + (x2, h2, rstd2)
        if self.cfg.remat == POLICY_SAVE_ATTENTION:
            return x3, (saved[3], saved[4])  # attention output and log-sum-exp only
        return x3, None

    # ------------------------------------------------------------------ layer backward
    def layer_backward(self, l: int, x: torch.Tensor, dx3: torch.Tensor, ctx: StepContext, saved=None):
        cfg, P = self.cfg, self.params
        B, S, H, D, d = ctx.B, ctx.S, self.H, self.D, cfg.d_model
        M = B * S
        if saved is None or len(saved) == 2:  # recompute the layer up to the FFN input (attention kept or not)
            x2, s = self._attn_block_fwd(l, x, ctx, kept_attn=saved)
            h2, rstd2 = K.rmsnorm_fwd(x2, P.w(f"l{l}.n2"), cfg.rms_eps)
            saved = s + (x2, h2, rstd2)
        h1, rstd1, qkv, attn, lse, x2, h2, rstd2 = saved
        # ---- blockwise FFN backward (each chunk recomputes its activations)
        dh2 = ffn.ffn_backward(_LayerFFNLinears(P, l), h2, dx3, cfg.ffn_chunk_size)
        dx2 = K.rmsnorm_bwd(dh2, x2, P.w(f"l{l}.n2"), rstd2, P.g(f"l{l}.n2"), dres=dx3)
        del dh2
        # ---- attention block backward
        attn2 = attn.view(M, d)
        dattn = P.lin_dgrad(dx2, f"l{l}.wo")
        P.lin_wgrad(dx2, attn2, f"l{l}.wo")
        qkv5 = qkv.view(B, S, 3, H, D)
        dqkv = torch.empty_like(qkv)
        dqkv5 = dqkv.view(B, S, 3, H, D)
        with phase("attn_bwd"):
            A.ring_backward(qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2], attn, lse, dattn.view(B, S, H, D),
                            ctx.plan, ctx.symm_ring, dq=dqkv5[:, :, 0], dk=dqkv5[:, :, 1], dv=dqkv5[:, :, 2])
        K.rope_(dqkv.view(B, S, 3 * H, D)[:, :, :2 * H], ctx.positions, cfg.rope_theta, inverse=True)
        P.lin_wgrad(dqkv, h1, f"l{l}.wqkv")
        dh1 = P.lin_dgrad(dqkv, f"l{l}.wqkv")
        dx = K.rmsnorm_bwd(dh1, x, P.w(f"l{l}.n1"), rstd1, P.g(f"l{l}.n1"), dres=dx2)
        return dx

    # ------------------------------------------------------------------ head (final norm + LM head + loss)
    def head_forward_backward(self, x: torch.Tensor, targets: torch.Tensor, ctx: StepContext,
                              compute_grad: bool = True):
        """Returns ``(sum of token losses on this rank, dx)``. The LM head runs in token chunks;
        each chunk's logits are turned into dlogits in place and consumed immediately."""
        cfg, P = self.cfg, self.params
        M = x.shape[0]
        hf, rstdf = K.rmsnorm_fwd(x, P.w("nf"), cfg.rms_eps)
        dhf = torch.empty_like(x) if compute_grad else None
        losses = torch.empty(M, device=x.device, dtype=torch.float32)
        step = min(cfg.loss_chunk_size, M)
        scale = 1.0 / max(1, ctx.total_tokens)
        tflat = targets.reshape(-1)
        for r0 in range(0, M, step):
            r1 = min(M, r0 + step)
            logits = P.lin_fwd(hf[r0:r1], "lm_head")
            K.xent_fwd_bwd_(logits, tflat[r0:r1], scale, loss=losses[r0:r1])
            if compute_grad:
                P.lin_wgrad(logits, hf[r0:r1], "lm_head")
                P.lin_dgrad(logits, "lm_head", out=dhf[r0:r1])
        loss_sum = losses.sum()
        if not compute_grad:
            return loss_sum, None
        dx = K.rmsnorm_bwd(dhf, x, P.w("nf"), rstdf, P.g("nf"))
        return loss_sum, dx

    # ------------------------------------------------------------------ full passes
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, ctx: StepContext):
        """One training forward+backward on this rank's shard. ``tokens``/``targets`` are
        ``(B, S_local)`` int32 (targets < 0 are ignored). Gradients are *added* to the flat fp32
        grad buffer; returns the local sum of token losses (a 0-d tensor)."""
        cfg, P = self.cfg, self.params
        P.ensure_grads()
        tok = tokens.reshape(-1).contiguous()
        x = K.embedding_fwd(tok, P.w("embed"))
        keep = cfg.remat not in (POLICY_NOTHING_SAVEABLE, POLICY_SAVE_ATTENTION)
        layer_inputs: List[torch.Tensor] = []
        saved_all: List[object] = []
        for l in range(cfg.n_layers):
            layer_inputs.append(x)
            x, saved = self.layer_forward(l, x, ctx, keep=keep)
            saved_all.append(saved)
        with phase("head"):
            loss_sum, dx = self.head_forward_backward(x, targets, ctx)
        del x
        for l in reversed(range(cfg.n_layers)):
            dx = self.layer_backward(l, layer_inputs[l], dx, ctx, saved_all[l])
            layer_inputs[l] = None
            saved_all[l] = None
        K.embedding_bwd(tok, dx, P.g("embed"))
        return loss_sum

    @torch.no_grad()
    def forward_loss(self, tokens, targets, ctx: StepContext):
        """Forward only; returns the local sum of token losses."""
        x = K.embedding_fwd(tokens.reshape(-1).contiguous(), self.params.w("embed"))
        for l in range(self.cfg.n_layers):
            x, _ = self.layer_forward(l, x, ctx)
        loss_sum, _ = self.head_forward_backward(x, targets, ctx, compute_grad=False)
        return loss_sum

    def flops_per_token(self, seq_len_global: int, causal: bool = True) -> float:
        """Model FLOPs per token for forward+backward (6 * matmul params + attention)."""
        cfg = self.cfg
        d, F, V = cfg.d_model, cfg.d_ff, cfg.vocab_size
        mm = cfg.n_layers * (4 * d * d + 3 * d * F) + V * d
        attn = cfg.n_layers * 2 * seq_len_global * d * (0.5 if causal else 1.0) * 2  # QK^T and PV
        return 6.0 * mm + 3.0 * attn
