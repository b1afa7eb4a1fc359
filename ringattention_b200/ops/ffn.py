"""Blockwise SwiGLU feed-forward on the sm_100a GEMM kernels.

``blockwise_feedforward`` of the reference (ringattention/ringattention_jax.py:333-352) scans a position-wise
feed-forward over sequence chunks under remat, so that only one chunk's ``(chunk, d_ff)`` activations exist
at a time. This module is the kernel-backed form of that loop for the SwiGLU feed-forward
``y = (silu(x Wg^T) * (x Wu^T)) Wd^T (+ residual)``:

* forward, per chunk: one GEMM against ``W = [Wg ; Wu]`` with the activation in its epilogue (the ``(chunk,
  2 d_ff)`` pre-activations never reach memory), one GEMM against ``Wd`` with the residual add in its epilogue;
* backward, per chunk: the pre-activations are recomputed (policy ``nothing_saveable``) or taken from the
  forward (``everything_saveable``), then ``dWd += dy^T a``, ``da = dy Wd``, the SwiGLU derivative in place,
  ``dW += dgu^T x`` and ``dx = dgu W`` - weight gradients accumulate in fp32 across chunks.

:func:`ffn_forward` / :func:`ffn_backward` take the linear layers as callables, so the LLaMA driver runs the
same loop on its flat, optionally fsdp-sharded parameters (``models/llama.py``). :class:`FusedSwiGLU` wraps them
in an ``nn.Module`` with autograd; ``ringattention_b200.blockwise_feedforward`` recognises it and runs its
chunks on the kernels instead of looping over a Python callable.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..config import POLICY_NOTHING_SAVEABLE, _policy_name
from . import kernels as K


class DenseLinears:
    """The four products of the feed-forward on plain ``(N, K)`` bf16 weight tensors."""

    def __init__(self, wgu: torch.Tensor, wd: torch.Tensor, dwgu: Optional[torch.Tensor] = None,
                 dwd: Optional[torch.Tensor] = None):
        self.wgu, self.wd, self.dwgu, self.dwd = wgu, wd, dwgu, dwd

    def gate_up(self, x):                      # (rows, 2F) pre-activations
        return K.linear_fwd(x, self.wgu)

    def gate_up_act(self, x):                  # (rows, F) = silu(gate) * up, activation in the GEMM epilogue
        return K.linear_swiglu(x, self.wgu)

    def down(self, a, out, residual):
        return K.linear_fwd(a, self.wd, out=out, residual=residual)

    def down_dgrad(self, dy):
        return K.linear_dgrad(dy, self.wd)

    def down_wgrad(self, dy, a):
        K.linear_wgrad(dy, a, self.dwd)

    def gate_up_wgrad(self, dgu, x):
        K.linear_wgrad(dgu, x, self.dwgu)

    def gate_up_dgrad(self, dgu, out):
        return K.linear_dgrad(dgu, self.wgu, out=out)


def ffn_forward(lin, x: torch.Tensor, chunk: int, residual: Optional[torch.Tensor] = None,
                keep: Optional[list] = None) -> torch.Tensor:
    """``x (rows, d)`` bf16 -> ``(rows, d)``, ``chunk`` rows at a time. ``keep``: a list that receives each
    chunk's pre-activations (for a backward without recomputation); then the two-pass path runs."""
    M = x.shape[0]
    y = torch.empty_like(x)
    step = min(chunk, M)
    for r0 in range(0, M, step):
        r1 = min(M, r0 + step)
        if keep is None:
            a = lin.gate_up_act(x[r0:r1])
        else:
            gu = lin.gate_up(x[r0:r1])
            keep.append(gu)
            a = K.swiglu_fwd(gu)
        lin.down(a, y[r0:r1], None if residual is None else residual[r0:r1])
    return y


def ffn_backward(lin, x: torch.Tensor, dy: torch.Tensor, chunk: int, kept: Optional[list] = None) -> torch.Tensor:
    """Returns ``dx``; weight gradients go through ``lin.down_wgrad`` / ``lin.gate_up_wgrad`` (fp32
    accumulation). ``kept``: pre-activations of the forward, else they are recomputed chunk by chunk."""
    M = x.shape[0]
    dx = torch.empty_like(x)
    step = min(chunk, M)
    for ci, r0 in enumerate(range(0, M, step)):
        r1 = min(M, r0 + step)
        gu = kept[ci] if kept is not None else lin.gate_up(x[r0:r1])
        a = K.swiglu_fwd(gu)
        da = lin.down_dgrad(dy[r0:r1])
        lin.down_wgrad(dy[r0:r1], a)
        K.swiglu_bwd_(gu, da)
        lin.gate_up_wgrad(gu, x[r0:r1])
        lin.gate_up_dgrad(gu, dx[r0:r1])
    return dx


class _BlockwiseSwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, wgu, wd, chunk, recompute):
        keep = None if recompute else []
        y = ffn_forward(DenseLinears(wgu, wd), x2, chunk, keep=keep)
        ctx.save_for_backward(x2, wgu, wd)
        ctx.chunk, ctx.kept = chunk, keep
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, wgu, wd = ctx.saved_tensors
        dy = dy.contiguous()
        dwgu = torch.zeros(wgu.shape, device=wgu.device, dtype=torch.float32)
        dwd = torch.zeros(wd.shape, device=wd.device, dtype=torch.float32)
        dx = ffn_backward(DenseLinears(wgu, wd, dwgu, dwd), x2, dy, ctx.chunk, kept=ctx.kept)
        ctx.kept = None
        return dx, dwgu.to(wgu.dtype), dwd.to(wd.dtype), None, None


class FusedSwiGLU(torch.nn.Module):
    """SwiGLU feed-forward whose chunks run on the tcgen05 GEMM kernels, with autograd.

    ``weight_gate_up`` is ``(2 * d_ff, d_model)`` (gate rows, then up rows), ``weight_down`` is ``(d_model,
    d_ff)``; both bf16 on a CUDA device. Calling the module applies it to ``(..., d_model)`` in one chunk;
    ``blockwise_feedforward(module, inputs, chunk_size, policy=...)`` applies it chunk by chunk with the
    policy's recomputation (``module.blockwise`` is what it calls)."""

    def __init__(self, d_model: int, d_ff: int, device="cuda", init_std: float = 0.02, seed: Optional[int] = None):
        super().__init__()
        if d_model % 8 or d_ff % 8:
            raise ValueError("d_model and d_ff must be multiples of 8")
        gen = None
        if seed is not None:
            gen = torch.Generator(device=device)
            gen.manual_seed(seed)
        self.d_model, self.d_ff = d_model, d_ff
        self.weight_gate_up = torch.nn.Parameter(
            (torch.randn(2 * d_ff, d_model, device=device, generator=gen) * init_std).bfloat16())
        self.weight_down = torch.nn.Parameter(
            (torch.randn(d_model, d_ff, device=device, generator=gen) * init_std).bfloat16())

    def blockwise(self, inputs: torch.Tensor, chunk_size: int, policy=POLICY_NOTHING_SAVEABLE) -> torch.Tensor:
        """``inputs (..., d_model)`` bf16; ``chunk_size`` tokens per chunk (of the flattened leading dims)."""
        if inputs.dtype != torch.bfloat16 or not inputs.is_cuda:
            raise ValueError("FusedSwiGLU takes CUDA bf16 inputs")
        x2 = inputs.reshape(-1, self.d_model).contiguous()
        recompute = _policy_name(policy) == POLICY_NOTHING_SAVEABLE
        y = _BlockwiseSwiGLU.apply(x2, self.weight_gate_up, self.weight_down, int(chunk_size), recompute)
        return y.view(inputs.shape)

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        rows = inputs.numel() // self.d_model
        return self.blockwise(inputs, max(1, rows))

    def reference(self, inputs: torch.Tensor) -> torch.Tensor:
        """The same function in plain PyTorch (fp32 math), for tests."""
        x = inputs.float()
        gu = x @ self.weight_gate_up.float().t()
        g, u = gu[..., :self.d_ff], gu[..., self.d_ff:]
        return (torch.nn.functional.silu(g) * u) @ self.weight_down.float().t()
