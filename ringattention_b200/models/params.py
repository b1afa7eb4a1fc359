"""Parameter storage of the LLaMA driver: flat buffers, optional row-sharding over an ``fsdp`` group.

All GEMM weights ``W[N][K]`` are split by rows into ``f`` shards of ``shard_rows = ceil(N/f/256)*256``
rows (``f = 1``: the whole matrix). The buffers are *shard-major*: the shard of rank r of every matrix
is contiguous, so the optimizer state a rank owns (fp32 master, moments) is one slice and AdamW is one
launch. Embedding table and norm gains are replicated.

With ``f > 1`` the bf16 working copy of a rank's shard lives in symmetric memory; the other ranks never
hold a gathered copy of the model. ``lin_fwd`` / ``lin_dgrad`` run the GEMM whose leading CTAs pull the
remote shards into a scratch while the rest of the grid already computes on the local rows
(``ringattention_b200/csrc/gemm_gather_sm100.cu``) - the parameter all-gather is fused into the GEMM that consumes the
weights. ``lin_wgrad`` produces the full weight gradient shard by shard; gradients are all-reduced by
the trainer and every rank applies only its own rows.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..config import LlamaConfig
from ..ops import _lib
from ..ops import kernels as K
from ..utils.tracing import phase

c_ll = ctypes.c_longlong
c_vp = ctypes.c_void_p


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class GatherSchedule:
    """Which gathered weight shards are resident, and what to copy during each sharded GEMM call.

    The landing area has two regions per kind of matrix (wqkv, wo, wgu, wd, lm_head). ``plan(name)``
    is called once per GEMM on matrix ``name`` and returns

    * ``region``: where the call reads the remote shards of ``name``;
    * ``copy_ctas``/``target``: ``gather_ctas`` and a new flag target when the shards must be pulled by
      this call (its tiles wait for them), else 0 and the target of the earlier pull;
    * ``prefetch``: for a call on resident shards, optionally ``(name2, region2, target2)``: the copy
      CTAs of this call pull matrix ``name2``, the first one the previous step needed after this
      point that is not resident, into a region no call before it reads.

    Flag targets count copy CTAs cumulatively (every pull adds ``gather_ctas`` to each remote shard's
    counter). The call sequence of a step is recorded; ``invalidate()`` (after the optimizer step)
    empties the regions and makes the recorded sequence the prediction for the next step. A wrong
    prediction only costs a later pull: correctness never depends on it."""

    def __init__(self, kinds, gather_ctas: int, prefetch: bool = True, window: int = 48):
        self.regions: Dict[str, List[Optional[list]]] = {k: [None, None] for k in kinds}  # [name, target, stamp]
        self.gather_ctas = gather_ctas
        self.prefetch = prefetch
        self.window = window
        self.flag_base = 0
        self.stamp = 0
        self.trace_prev: List[str] = []
        self.trace_cur: List[str] = []
        self.trace_ok = True
        self.stats = {"gathers": 0, "prefetches": 0, "resident_calls": 0}

    @staticmethod
    def kind(name: str) -> str:
        return name.split(".")[-1]

    def find(self, name: str) -> int:
        regs = self.regions[self.kind(name)]
        for r in (0, 1):
            if regs[r] is not None and regs[r][0] == name:
                return r
        return -1

    def _next_miss(self, i: int, current: str):
        prev = self.trace_prev
        if not (self.prefetch and self.trace_ok and i < len(prev)):
            return None
        needed = {current}                             # the running call still reads its own shards
        for j in range(i + 1, min(len(prev), i + 1 + self.window)):
            nm = prev[j]
            if self.find(nm) >= 0:
                needed.add(nm)
                continue
            regs = self.regions[self.kind(nm)]
            free = [r for r in (0, 1) if regs[r] is None or regs[r][0] not in needed]
            if not free:
                return None
            free.sort(key=lambda r: -1 if regs[r] is None else regs[r][2])  # empty first, then least recent
            return nm, free[0]
        return None

    def plan(self, name: str) -> dict:
        regs = self.regions[self.kind(name)]
        i = len(self.trace_cur)
        self.trace_cur.append(name)
        if self.trace_ok and i < len(self.trace_prev) and self.trace_prev[i] != name:
            self.trace_ok = False                      # this step differs from the last one: no predictions
        self.stamp += 1
        r = self.find(name)
        if r >= 0:
            regs[r][2] = self.stamp
            self.stats["resident_calls"] += 1
            out = {"region": r, "copy_ctas": 0, "target": regs[r][1], "prefetch": None}
            nxt = self._next_miss(i, name)
            if nxt is not None:
                nm2, r2 = nxt
                self.flag_base += self.gather_ctas
                self.regions[self.kind(nm2)][r2] = [nm2, self.flag_base, self.stamp]
                out["copy_ctas"] = self.gather_ctas
                out["prefetch"] = (nm2, r2, self.flag_base)
                self.stats["prefetches"] += 1
            return out
        r = min((0, 1), key=lambda q: -1 if regs[q] is None else regs[q][2])
        self.flag_base += self.gather_ctas
        regs[r] = [name, self.flag_base, self.stamp]
        self.stats["gathers"] += 1
        return {"region": r, "copy_ctas": self.gather_ctas, "target": self.flag_base, "prefetch": None}

    def invalidate(self) -> None:
        for regs in self.regions.values():
            regs[0] = regs[1] = None
        self.trace_prev, self.trace_cur, self.trace_ok = self.trace_cur, [], True


class FlatParams:
    def __init__(self, cfg: LlamaConfig, device, seed: int = 0, with_optimizer: bool = True,
                 shard: Tuple[int, int] = (0, 1), fsdp_group=None, gather_ctas: int = 16, zero=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.shard_index, self.shard_count = shard
        self.zero = zero if (zero is not None and zero[1] > 1) else None
        zc = self.zero[1] if self.zero else 1
        self.fsdp_group = fsdp_group
        self.gather_ctas = gather_ctas
        f = self.shard_count
        d, F, V = cfg.d_model, cfg.d_ff, cfg.vocab_size

        # ---- layout
        self.mat: Dict[str, Tuple[int, int, int, int]] = {}   # name -> (offset in shard, N, K, shard_rows)
        self.rep: Dict[str, Tuple[int, Tuple[int, ...]]] = {}  # name -> (offset in replicated region, shape)
        off = 0
        mats: List[Tuple[str, int, int]] = []
        for l in range(cfg.n_layers):
            mats += [(f"l{l}.wqkv", 3 * d, d), (f"l{l}.wo", d, d), (f"l{l}.wgu", 2 * F, d), (f"l{l}.wd", d, F)]
        mats.append(("lm_head", V, d))
        for name, N, Kd in mats:
            sr = N if f == 1 else _round_up((N + f - 1) // f, 256)
            self.mat[name] = (off, N, Kd, sr)
            off += _round_up(sr * Kd, 64)
        self.numel_shard = _round_up(off, 1024 * zc)
        off = 0
        self.rep["embed"] = (off, (V, d))
        off += _round_up(V * d, 64)
        self.rep_decay_end = off
        for l in range(cfg.n_layers):
            for nm in (f"l{l}.n1", f"l{l}.n2"):
                self.rep[nm] = (off, (d,))
                off += _round_up(d, 64)
        self.rep["nf"] = (off, (d,))
        off += _round_up(d, 64)
        self.numel_rep = _round_up(off, 1024 * zc)
        self.index = {**{n: None for n in self.mat}, **{n: None for n in self.rep}}

        # ---- storage
        self._symm = None
        if f > 1:
            from ..parallel.symm import SymmBuffer

            self._symm = SymmBuffer(self.numel_shard * 2, fsdp_group, self.device)
            self.p16_shard = self._symm.local.view(torch.bfloat16)[:self.numel_shard]
            # Landing area of gathered remote shards: two regions per kind of matrix (wqkv, wo, wgu, wd,
            # lm_head), each holding the f-1 remote shards of ONE matrix of that kind. A matrix stays
            # resident until its region is reused, so the chunk loops of the feed-forward and of the LM
            # head, and the backward right after the recomputation of a layer, reuse the copy; the
            # second region lets a call on resident shards prefetch the matrix that the previous step
            # needed next (the sequence of calls repeats from step to step).
            self._kind_off: Dict[str, int] = {}
            self._kind_size: Dict[str, int] = {}
            tot = 0
            for name, (_, _, Kd, sr) in self.mat.items():
                kind = name.split(".")[-1]
                if kind not in self._kind_off:
                    self._kind_off[kind] = tot
                    self._kind_size[kind] = _round_up(sr * Kd, 64)
                    tot += 2 * (f - 1) * self._kind_size[kind]
            self._scratch = torch.empty(tot, device=self.device, dtype=torch.bfloat16)
            self.sched = GatherSchedule(self._kind_off.keys(), self.gather_ctas)
            self._flags = torch.zeros(8, dtype=torch.int32, device=self.device)
        else:
            self.p16_shard = torch.empty(self.numel_shard, device=self.device, dtype=torch.bfloat16)
        self.p16_rep = torch.empty(self.numel_rep, device=self.device, dtype=torch.bfloat16)
        self.g32: Optional[torch.Tensor] = None
        self._init_weights(seed)
        self.p32_s = self.m_s = self.v_s = self.p32_r = self.m_r = self.v_r = None
        if with_optimizer:
            self.p32_s = self.own(self.p16_shard).float()
            self.m_s = torch.zeros_like(self.p32_s)
            self.v_s = torch.zeros_like(self.p32_s)
            self.p32_r = self.own(self.p16_rep).float()
            self.m_r = torch.zeros_like(self.p32_r)
            self.v_r = torch.zeros_like(self.p32_r)
        if f > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=fsdp_group)

    # ------------------------------------------------------------------ init
    def _init_weights(self, seed: int) -> None:
        """N(0, init_std) per tensor from a generator seeded by (seed, tensor index): the values do
        not depend on the sharding."""
        cfg = self.cfg
        self.p16_shard.zero_()
        self.p16_rep.zero_()
        gen = torch.Generator(device=self.device)
        for ti, (name, (off, N, Kd, sr)) in enumerate(self.mat.items()):
            gen.manual_seed(seed * 100003 + ti)
            r0 = self.shard_index * sr
            r1 = min(N, r0 + sr)
            full = torch.randn(N, Kd, device=self.device, generator=gen) * cfg.init_std
            if r1 > r0:
                self.p16_shard[off:off + (r1 - r0) * Kd].view(r1 - r0, Kd).copy_(full[r0:r1])
            del full
        gen.manual_seed(seed * 100003 + 99991)
        eoff, eshape = self.rep["embed"]
        self.p16_rep[eoff:eoff + math.prod(eshape)].view(eshape).copy_(
            torch.randn(*eshape, device=self.device, generator=gen) * cfg.init_std)
        for name, (off, shape) in self.rep.items():
            if len(shape) == 1:
                self.p16_rep[off:off + shape[0]] = 1.0

    # ------------------------------------------------------------------ views
    def own(self, region: torch.Tensor) -> torch.Tensor:
        """The slice of a flat region (shard region or replicated tail, of any dtype) whose optimizer state
        this rank keeps: all of it unless the state is sharded over the replicas."""
        if self.zero is None:
            return region
        zi, zc, _ = self.zero
        n = region.numel() // zc
        return region[zi * n:(zi + 1) * n]

    @property
    def numel_grads(self) -> int:
        return self.shard_count * self.numel_shard + self.numel_rep

    def ensure_grads(self) -> torch.Tensor:
        if self.g32 is None:
            self.g32 = torch.zeros(self.numel_grads, device=self.device, dtype=torch.float32)
        return self.g32

    def grad_shard(self, s: int) -> torch.Tensor:
        return self.g32[s * self.numel_shard:(s + 1) * self.numel_shard]

    def grad_rep(self) -> torch.Tensor:
        return self.g32[self.shard_count * self.numel_shard:]

    def w(self, name: str) -> torch.Tensor:
        """Replicated tensors always; matrices only when they are not sharded."""
        if name in self.rep:
            off, shape = self.rep[name]
            return self.p16_rep[off:off + math.prod(shape)].view(shape)
        off, N, Kd, sr = self.mat[name]
        if self.shard_count != 1:
            raise RuntimeError(f"{name} is sharded over {self.shard_count} ranks; use lin_fwd/lin_dgrad")
        return self.p16_shard[off:off + N * Kd].view(N, Kd)

    def w_shard(self, name: str) -> torch.Tensor:
        """This rank's rows of a matrix (``(rows, K)``; the last shard may be shorter)."""
        off, N, Kd, sr = self.mat[name]
        rows = max(0, min(sr, N - self.shard_index * sr))
        return self.p16_shard[off:off + rows * Kd].view(rows, Kd)

    def g(self, name: str) -> torch.Tensor:
        if name in self.rep:
            off, shape = self.rep[name]
            return self.grad_rep()[off:off + math.prod(shape)].view(shape)
        off, N, Kd, sr = self.mat[name]
        if self.shard_count != 1:
            raise RuntimeError(f"{name} is sharded; its gradient is stored shard by shard")
        return self.g32[off:off + N * Kd].view(N, Kd)

    def g_full(self, name: str) -> torch.Tensor:
        """Gradient of a matrix assembled to ``(N, K)`` (a copy when sharded; for tests)."""
        if name in self.rep or self.shard_count == 1:
            return self.g(name)
        off, N, Kd, sr = self.mat[name]
        parts = []
        for s in range(self.shard_count):
            rows = max(0, min(sr, N - s * sr))
            parts.append(self.grad_shard(s)[off:off + rows * Kd].view(rows, Kd))
        return torch.cat(parts, dim=0)

    def n_params(self) -> int:
        return sum(N * Kd for (_, N, Kd, _) in self.mat.values()) + sum(math.prod(s) for _, s in self.rep.values())

    def invalidate_gathered(self) -> None:
        """Forget which remote shards are resident (call whenever any rank's weights change)."""
        if self.shard_count > 1:
            self.sched.invalidate()

    # ------------------------------------------------------------------ linear layers
    def _region_ptrs(self, name: str, region: int):
        """Per shard: local address the GEMM reads, and the owner's address (0 for the own shard)."""
        off, Nw, Kw, sr = self.mat[name]
        kind = name.split(".")[-1]
        f, me = self.shard_count, self.shard_index
        base = self._kind_off[kind] + region * (f - 1) * self._kind_size[kind]
        local_ptrs, src_ptrs, n16 = [], [], []
        slot = 0
        for s in range(f):
            rows = max(0, min(sr, Nw - s * sr))
            if s == me:
                local_ptrs.append(self.p16_shard.data_ptr() + off * 2)
                src_ptrs.append(0)
                n16.append(0)
            else:
                local_ptrs.append(self._scratch.data_ptr() + (base + slot * self._kind_size[kind]) * 2)
                src_ptrs.append(self._symm.peer_ptrs[s] + off * 2)
                n16.append(rows * Kw * 2 // 16)
                slot += 1
        return local_ptrs, src_ptrs, n16

    def _gather_call(self, x, name, b_mn: int, out, residual, M, N, Kg):
        off, Nw, Kw, sr = self.mat[name]
        f, me = self.shard_count, self.shard_index
        plan = self.sched.plan(name)
        PF_D = PF_S = PF_N = None
        if plan["prefetch"] is not None:
            nm2, r2, _ = plan["prefetch"]
            d2, s2, n2 = self._region_ptrs(nm2, r2)
            PF_D, PF_S, PF_N = (c_vp * f)(*d2), (c_vp * f)(*s2), (c_ll * f)(*n2)
        local_ptrs, src_ptrs, _ = self._region_ptrs(name, plan["region"])
        LP = (c_vp * f)(*local_ptrs)
        SP = (c_vp * f)(*src_ptrs)
        c_fp32 = 1 if out.dtype == torch.float32 else 0
        _lib.call("ra_gemm_bf16_gather", c_vp(x.data_ptr()), c_vp(out.data_ptr()),
                  c_vp(0 if residual is None else residual.data_ptr()), M, N, Kg,
                  c_ll(x.stride(0)), c_ll(out.stride(0)), c_ll(0 if residual is None else residual.stride(0)),
                  b_mn, c_fp32, f, me, sr, c_ll(Kw), LP, SP, c_vp(self._flags.data_ptr()),
                  ctypes.c_uint(plan["target"] & 0xFFFFFFFF), plan["copy_ctas"], 8,
                  c_vp(_lib.status_tensor(self.device).data_ptr()), _lib.stream_ptr(), PF_D, PF_S, PF_N)
        return out

    @property
    def gather_stats(self) -> dict:
        return self.sched.stats if self.shard_count > 1 else {}

    def lin_fwd(self, x, name: str, out=None, residual=None):
        """``y = x W^T (+ residual)``."""
        off, N, Kd, sr = self.mat[name]
        with phase("linear"):
            if self.shard_count == 1:
                return K.linear_fwd(x, self.w(name), out=out, residual=residual)
            M = x.shape[0]
            if out is None:
                out = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
            return self._gather_call(x, name, 0, out, residual, M, N, Kd)

    def lin_dgrad(self, dy, name: str, out=None, residual=None):
        """``dx = dy W (+ residual)``."""
        off, N, Kd, sr = self.mat[name]
        with phase("linear"):
            if self.shard_count == 1:
                return K.linear_dgrad(dy, self.w(name), out=out, residual=residual)
            M = dy.shape[0]
            if out is None:
                out = torch.empty(M, Kd, device=dy.device, dtype=torch.bfloat16)
            return self._gather_call(dy, name, 1, out, residual, M, Kd, N)

    def lin_wgrad(self, dy, x, name: str) -> None:
        """``dW += dy^T x`` (fp32). With sharding, each shard's rows are a GEMM of their own, written
        into that shard's segment of the gradient buffer."""
        off, N, Kd, sr = self.mat[name]
        with phase("wgrad"):
            if self.shard_count == 1:
                K.linear_wgrad(dy, x, self.g(name))
                return
            for s in range(self.shard_count):
                r0 = s * sr
                rows = max(0, min(sr, N - r0))
                if rows == 0:
                    continue
                acc = self.grad_shard(s)[off:off + rows * Kd].view(rows, Kd)
                K.gemm(dy[:, r0:r0 + rows], x, a_mn=True, b_mn=True, out=acc, residual=acc)

    # ------------------------------------------------------------------ optimizer
    def adamw_step(self, step: int, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
                   clip: float, gnorm_sq) -> None:
        common = dict(step=step, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                      clip=clip, gnorm_sq=gnorm_sq)
        self.invalidate_gathered()
        rep_start = 0 if self.zero is None else self.zero[0] * (self.numel_rep // self.zero[1])
        rep_decay = max(0, min(self.p32_r.numel(), self.rep_decay_end - rep_start))
        K.adamw_(self.p32_s, self.m_s, self.v_s, self.own(self.grad_shard(self.shard_index)),
                 self.own(self.p16_shard), decay_end=self.p32_s.numel(), **common)
        K.adamw_(self.p32_r, self.m_r, self.v_r, self.own(self.grad_rep()), self.own(self.p16_rep),
                 decay_end=rep_decay, **common)
        self.gather_working_copy()

    def gather_working_copy(self) -> None:
        """With optimizer state sharded over the replicas, every rank has just updated its slice of the bf16
        weights: all-gather the slices (in place) so that each rank holds its full shard region and tail."""
        if self.zero is None:
            return
        from ..parallel import gradsync

        zi, zc, zg = self.zero
        with phase("param_allgather"):
            gradsync.all_gather_(self.p16_shard, zi, zc, zg)
            gradsync.all_gather_(self.p16_rep, zi, zc, zg)

    def state_dict(self) -> dict:
        return {"p32_s": self.p32_s.cpu(), "m_s": self.m_s.cpu(), "v_s": self.v_s.cpu(),
                "p32_r": self.p32_r.cpu(), "m_r": self.m_r.cpu(), "v_r": self.v_r.cpu(),
                "shard": (self.shard_index, self.shard_count),
                "zero": (0, 1) if self.zero is None else (self.zero[0], self.zero[1])}

    def load_state_dict(self, st: dict) -> None:
        if tuple(st["shard"]) != (self.shard_index, self.shard_count):
            raise ValueError("checkpoint was written with a different fsdp sharding")
        mine = (0, 1) if self.zero is None else (self.zero[0], self.zero[1])
        if tuple(st.get("zero", (0, 1))) != mine:
            raise ValueError("checkpoint was written with a different sharding of the optimizer state")
        self.invalidate_gathered()
        for k in ("p32_s", "m_s", "v_s", "p32_r", "m_r", "v_r"):
            getattr(self, k).copy_(st[k])
        self.own(self.p16_shard).copy_(self.p32_s)
        self.own(self.p16_rep).copy_(self.p32_r)
        self.gather_working_copy()
