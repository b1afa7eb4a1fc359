"""Long-context inference on the LLaMA driver: sequence-sharded KV cache, chunked prefill and
greedy decoding.

The reference's inference contract gives rank r of the ``sp`` axis a contiguous range of positions
(ringattention_inference.py:19-20, ringattention_jax.py:34-35) and rotates the whole cache for every
call. Here the cache never moves and is *striped*: every prefill chunk leaves the slice a rank
computed on that rank, so all ranks hold equally many rows at any time (with contiguous ranges the
ranks that own late positions idle through most of the prefill: 13.3K tokens/s on 8 GPUs at 1M
tokens). Rows are kept in arrival order; attention over past rows needs no positions, only the rows
of the chunk being prefilled are masked causally at their true positions.

* prefill: the chunk's tokens are split over the ranks for the dense layers; each rank keeps its own
  K/V slice; queries are all-gathered (small), every rank runs the flash kernel against *its own*
  cache rows, and the per-rank ``(o, lse)`` partials are exchanged and merged. Both exchanges are peer
  stores into symmetric buffers followed by a flag barrier; the only library collective of a prefill
  chunk is the final broadcast of the logits;
* decode: the tiny dense layers are computed redundantly on every rank (weights are replicated), the
  new token's K/V go to rank ``i % N`` (i = index of the decoded token), attention runs the split-KV
  kernel on the local rows and merges across GPUs through peer stores.
"""
from __future__ import annotations

import ctypes
import time
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config import LlamaConfig
from ..ops import _lib
from ..ops import decode as Dk
from ..ops import ffn
from ..ops import flash
from ..ops import kernels as K
from ..ops.flash import MaskSpec, Positions
from ..parallel.mesh import AxisContext, resolve_axis
from .llama import _LayerFFNLinears
from .params import FlatParams


class LlamaInference:
    def __init__(self, cfg: LlamaConfig, max_context: int, batch: int = 1, device="cuda", seed: int = 0,
                 axis: "AxisContext | str | None" = None, params: Optional[FlatParams] = None,
                 symm_ring=None, streams: int = 0, max_new_tokens: int = 512):
        """``streams > 0``: one cached context (``batch`` must be 1) shared by that many decode streams (at most
        8). The prefix is prefilled once and read once per decoded step for all streams; every stream keeps the
        K/V of its own decoded tokens in a small private tail (``max_new_tokens`` long, striped over the ranks).
        This is how a batch of long-context requests fits when distinct contexts do not: four 1M-token contexts
        of the 7B model would need 2 TiB of KV."""
        self.cfg = cfg
        if streams and (batch != 1 or not 1 <= streams <= 8):
            raise ValueError("shared-prefix decoding takes batch = 1 and 1..8 streams")
        self.streams = int(streams)
        self.device = torch.device(device)
        self.axis = resolve_axis(axis)
        self.rank, self.world = self.axis.rank, self.axis.size
        self.group = self.axis.group
        self.symm_ring = symm_ring
        if self.world > 1 and symm_ring is None:
            from ..parallel.symm import SymmRing

            self.symm_ring = SymmRing(self.group, self.device)
        self.params = params if params is not None else FlatParams(cfg, self.device, seed, with_optimizer=False)
        self.B = batch
        self.H, self.D, self.d = cfg.n_heads, cfg.head_dim, cfg.d_model
        if max_context % (self.world * 128):
            raise ValueError("max_context must be a multiple of 128 * sp")
        self.S_max = max_context // self.world      # cache rows per rank
        # Striped cache: every prefill chunk leaves 1/N of its tokens on every rank (the slice the rank
        # computed itself), so all ranks hold equally many rows at any time and the attention work of
        # every later chunk is balanced; decoded tokens are dealt round-robin. Rows are in arrival order;
        # only rows of the chunk being prefilled need their true positions (causal rule inside the chunk).
        self.n_rows = 0                             # local rows written by prefill
        self.prefill_len = 0                        # positions covered by prefill
        # Heads-major storage (B, 2, H, S_max, D): the rows of one (k|v, head) are contiguous, so every CTA of the
        # split-KV decode kernel streams one long run instead of 256-byte pieces 16 KB apart. The kernels see
        # (B, S_max, H, D) views with strides; the flash kernel's tensor maps and the decode kernel take any strides.
        self._cache = [torch.zeros(batch, 2, self.H, self.S_max, self.D, device=self.device, dtype=torch.bfloat16)
                       for _ in range(cfg.n_layers)]
        self.k_cache = [c[:, 0].permute(0, 2, 1, 3) for c in self._cache]   # (B, S_max, H, D) views
        self.v_cache = [c[:, 1].permute(0, 2, 1, 3) for c in self._cache]
        self.length = 0                             # tokens in the cache (global)
        # [position, step] on the device: lets one recorded CUDA graph serve every decode step
        self.state = torch.zeros(2, dtype=torch.int64, device=self.device)
        self._graph = None
        self._xchg = 0                              # prefill exchanges so far (parity picks the peer-memory buffer)
        self._tok_buf = torch.zeros(max(batch, self.streams), dtype=torch.int32, device=self.device)
        if self.streams:
            t_tail = (max_new_tokens + self.world - 1) // self.world + 1
            self._tail = [torch.zeros(self.streams, 2, self.H, t_tail, self.D, device=self.device, dtype=torch.bfloat16)
                          for _ in range(cfg.n_layers)]
            self.k_tail = [c[:, 0].permute(0, 2, 1, 3) for c in self._tail]  # (streams, T, H, D) views
            self.v_tail = [c[:, 1].permute(0, 2, 1, 3) for c in self._tail]
            self._sp_work = [dict() for _ in range(cfg.n_layers)]
        self._logits_buf = None

    # ------------------------------------------------------------------ helpers
    def _rows_to(self, src: torch.Tensor, dst_ptr: int, rows: int, row_bytes: int, src_ld: int, dst_ld: int) -> None:
        """Strided row copy whose destination may be a peer's memory (plain stores over NVLink)."""
        _lib.call("ra_copy_rows", ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst_ptr), ctypes.c_longlong(rows),
                  ctypes.c_longlong(row_bytes), ctypes.c_longlong(src_ld), ctypes.c_longlong(dst_ld), _lib.stream_ptr())

    def _gather_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """All-gather of a ``(B, t, H, D)`` bf16 tensor along the token dim over the sp axis through peer memory:
        every rank stores its slice into slot ``rank`` of each peer's ``(B, N*t, H, D)`` buffer and a flag
        barrier orders the stores before the read. Two buffers alternate, so a rank that is already one exchange
        ahead never writes into a buffer its peer still reads (it cannot be two ahead: the barrier in between
        needs that peer)."""
        if self.world == 1:
            return x
        N, ring = self.world, self.symm_ring
        B, t, H, D = x.shape
        x = x.contiguous()
        nb = B * N * t * H * D * 2
        buf = ring.buffer("prefill_q_all", 2 * nb)
        slot = self._xchg & 1
        row = t * H * D * 2                                   # one batch row of one rank's slice, in bytes
        for r in range(N):
            self._rows_to(x, buf.peer_ptrs[r] + slot * nb + self.rank * row, B, row, row, N * row)
        ring.barrier()
        return buf.local[slot * nb:(slot + 1) * nb].view(torch.bfloat16).view(B, N * t, H, D)

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill_chunk(self, tokens: torch.Tensor) -> torch.Tensor:
        """Append a chunk ``tokens (B, Tc)`` (identical on all ranks, ``Tc`` divisible by 128*sp) to
        the cache. Returns the last position's logits ``(B, vocab)`` fp32 on every rank."""
        cfg, P = self.cfg, self.params
        B, Tc = tokens.shape
        N, H, D, d = self.world, self.H, self.D, self.d
        if Tc % (N * 128):
            raise ValueError("chunk length must be a multiple of 128 * sp")
        t = Tc // N
        pos0 = self.length
        if self.prefill_len != self.length:
            raise RuntimeError("prefill after decode is not supported by the striped cache")
        n0 = self.n_rows
        if n0 + t > self.S_max:
            raise ValueError("context exceeds max_context")
        mypos = Positions(pos0 + self.rank * t)
        tok = tokens[:, self.rank * t:(self.rank + 1) * t].to(self.device, torch.int32).contiguous()
        x = K.embedding_fwd(tok.reshape(-1), P.w("embed"))
        # keys: rows [0, n0) are earlier chunks (any position below pos0 serves the causal rule), rows
        # [n0, n0 + t) are this rank's slice of the chunk at its true positions
        k_pos = Positions(pos0 + self.rank * t) if n0 == 0 else Positions(0, pos0 + self.rank * t, n0)
        for l in range(cfg.n_layers):
            h1, _ = K.rmsnorm_fwd(x, P.w(f"l{l}.n1"), cfg.rms_eps)
            qkv = P.lin_fwd(h1, f"l{l}.wqkv")
            K.rope_(qkv.view(B, t, 3 * H, D)[:, :, :2 * H], mypos, cfg.rope_theta)
            qkv5 = qkv.view(B, t, 3, H, D)
            kc, vc = self.k_cache[l], self.v_cache[l]
            kc[:, n0:n0 + t].copy_(qkv5[:, :, 1])                            # own K/V slice stays local
            vc[:, n0:n0 + t].copy_(qkv5[:, :, 2])
            q_all = self._gather_tokens(qkv5[:, :, 0].contiguous())          # (B, Tc, H, D)
            ms = MaskSpec(causal_block_size=cfg.causal_block_size, q_pos=Positions(pos0), k_pos=k_pos)
            o_p, lse_p = flash.flash_fwd(q_all, kc[:, :n0 + t], vc[:, :n0 + t], ms, out_fp32=(N > 1))
            if N == 1:
                attn = o_p
            else:
                attn = self._merge_prefill(o_p, lse_p, t)
            x = P.lin_fwd(attn.reshape(B * t, d), f"l{l}.wo", residual=x)
            h2, _ = K.rmsnorm_fwd(x, P.w(f"l{l}.n2"), cfg.rms_eps)
            x = ffn.ffn_forward(_LayerFFNLinears(P, l), h2, cfg.ffn_chunk_size, residual=x)
        self.length = self.prefill_len = pos0 + Tc
        self.n_rows = n0 + t
        # logits of the globally last token live on the last rank; share them
        last = x.view(B, t, d)[:, -1].contiguous()
        hf, _ = K.rmsnorm_fwd(last, P.w("nf"), cfg.rms_eps)
        logits = K.small_m_linear(hf, P.w("lm_head")).float() if B <= 8 else K.linear_fwd(hf, P.w("lm_head")).float()
        if N > 1:
            dist.broadcast(logits, dist.get_global_rank(self.group, N - 1), group=self.group)
        return logits

    def _merge_prefill(self, o_p: torch.Tensor, lse_p: torch.Tensor, t: int) -> torch.Tensor:
        """Every rank holds a partial ``(o, lse)`` of all ``N*t`` query rows against its own cache rows; rank r
        needs the N partials of rows ``[r*t, (r+1)*t)``. Each rank stores those rows of its partial straight into
        slot ``rank`` of rank r's inbox (peer stores), a flag barrier follows, and the log-sum-exp kernel merges
        the N slots. Two inboxes alternate from exchange to exchange, as in :meth:`_gather_tokens`."""
        N, B, H, D, ring = self.world, o_p.shape[0], self.H, self.D, self.symm_ring
        lse_bth = lse_p.permute(0, 2, 1).contiguous()                          # (B, N*t, H), rows like o_p
        rows = B * t * H
        n_o, n_l = N * rows * D * 4, N * rows * 4                                # bytes per inbox
        box_o = ring.buffer("prefill_inbox_o", 2 * n_o)
        box_l = ring.buffer("prefill_inbox_lse", 2 * n_l)
        slot = self._xchg & 1
        self._xchg += 1
        ro, rl = t * H * D * 4, t * H * 4                                        # bytes of one batch row per dest
        for r in range(N):
            self._rows_to(o_p.view(B, N, t * H * D)[:, r], box_o.peer_ptrs[r] + slot * n_o + self.rank * B * ro,
                          B, ro, N * ro, ro)
            self._rows_to(lse_bth.view(B, N, t * H)[:, r], box_l.peer_ptrs[r] + slot * n_l + self.rank * B * rl,
                          B, rl, N * rl, rl)
        ring.barrier()
        recv_o = box_o.local[slot * n_o:(slot + 1) * n_o].view(torch.float32).view(N, rows, D)
        recv_l = box_l.local[slot * n_l:(slot + 1) * n_l].view(torch.float32).view(N, rows)
        out = torch.empty(B, t, H, D, device=self.device, dtype=torch.bfloat16)
        Dk.merge_partials(recv_o.permute(1, 0, 2), recv_l.permute(1, 0), H, 0, out=out)
        return out

    # ------------------------------------------------------------------ decode
    def _decode_body(self, tokens: torch.Tensor) -> torch.Tensor:
        """All launches of one decode step. Every per-token scalar (position, valid cache rows, inbox
        slot, barrier count) is read from device memory, so the sequence can be graph-captured."""
        cfg, P = self.cfg, self.params
        B, H, D, d = (self.streams or self.B), self.H, self.D, self.d
        stripe = (self.world, self.rank, self.n_rows, self.prefill_len)
        tail_stripe = (self.world, self.rank, 0, self.prefill_len)
        x = K.embedding_fwd(tokens, P.w("embed"))
        for l in range(cfg.n_layers):
            # RMSNorm runs in the prologue of the projection, RoPE and the cache append share a launch, and
            # SwiGLU runs in the prologue of the down projection: 7 launches per layer instead of 11 (13 on a ring)
            qkv = K.norm_linear(x, P.w(f"l{l}.n1"), cfg.rms_eps, P.w(f"l{l}.wqkv"))
            q = qkv.view(B, 1, 3, H, D)[:, :, 0]
            if self.streams:  # shared prefix: the new K/V go to the streams' private tails
                K.rope_append(qkv, self.k_tail[l], self.v_tail[l], self.state, cfg.rope_theta, stripe=tail_stripe)
                attn = Dk.shared_prefix_decode_attention(
                    q.contiguous(), self.k_cache[l], self.v_cache[l], self.n_rows, self.k_tail[l], self.v_tail[l],
                    self.axis, self.symm_ring, state=self.state, stripe=tail_stripe, exchange=l,
                    exchanges_per_step=cfg.n_layers, work=self._sp_work[l])
            else:
                K.rope_append(qkv, self.k_cache[l], self.v_cache[l], self.state, cfg.rope_theta, stripe=stripe)
                attn = Dk.ring_decode_attention(q.contiguous(), self.k_cache[l], self.v_cache[l],
                                                None, self.axis, self.symm_ring, k_pos0=0, state=self.state,
                                                exchange=l, exchanges_per_step=cfg.n_layers, stripe=stripe)
            x = K.linear_auto(attn.reshape(B, d), P.w(f"l{l}.wo"), residual=x)
            gu = K.norm_linear(x, P.w(f"l{l}.n2"), cfg.rms_eps, P.w(f"l{l}.wgu"))
            x = K.swiglu_linear(gu, P.w(f"l{l}.wd"), residual=x)
        logits = K.norm_linear(x, P.w("nf"), cfg.rms_eps, P.w("lm_head")).float()
        K.decode_advance(self.state)
        return logits

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """One token per sequence: ``tokens (B,)`` -> logits ``(B, vocab)`` fp32 (same on all ranks)."""
        self.state[0] = self.length
        logits = self._decode_body(tokens.to(self.device, torch.int32).reshape(-1).contiguous())
        self.length += 1
        return logits

    @torch.no_grad()
    def decode_step_graph(self) -> torch.Tensor:
        """Greedy step on the token in ``self._tok_buf`` through a CUDA graph recorded on first use:
        one replay per token instead of 7 launches per layer. Writes the next token back into
        ``self._tok_buf`` and returns it. Call :meth:`decode_step` at least once before (buffers and
        kernels must exist before capture)."""
        if self._graph is None:
            self.state[0] = self.length
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                logits = self._decode_body(self._tok_buf)
                self._tok_buf.copy_(logits.argmax(dim=-1).to(torch.int32))
            self._graph = g
        self._graph.replay()
        self.length += 1
        return self._tok_buf

    def reset(self) -> None:
        """Forget the cached context (the cache memory is kept). The recorded decode graph is dropped
        too: it holds the row count and length of the prefilled context as launch constants."""
        self.length = self.n_rows = self.prefill_len = 0
        self.state.zero_()
        self._graph = None

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, new_tokens: int, chunk: int = 32768, use_graph: bool = True):
        """Chunked prefill of ``prompt (B, T)`` followed by greedy decoding. Returns the generated
        tokens ``(B, new_tokens)`` and timing: prefill seconds, per-token decode latencies."""
        B, T = prompt.shape
        if self.length:
            self.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        logits = None
        for c0 in range(0, T, chunk):
            logits = self.prefill_chunk(prompt[:, c0:c0 + chunk])
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        out: List[torch.Tensor] = []
        lat: List[float] = []
        nxt = logits.argmax(dim=-1)
        if self.streams:  # the streams start from the `streams` most likely continuations of the shared prefix
            nxt = logits[0].topk(self.streams).indices
        for i in range(new_tokens):
            out.append(nxt.clone())
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if use_graph and i >= 2:
                if i == 2:
                    self._tok_buf.copy_(nxt.to(torch.int32))
                nxt = self.decode_step_graph()
            else:
                nxt = self.decode_step(nxt).argmax(dim=-1)
            e1.record()
            torch.cuda.synchronize()
            lat.append(e0.elapsed_time(e1))
        return torch.stack([t.to(torch.int64) for t in out], dim=1), {"prefill_s": t_prefill, "decode_ms": lat}
