"""Training engine: process-group / mesh bring-up, synthetic and packed-document data, the
training step (H2D -> forward/backward -> gradient all-reduce -> clip + AdamW -> loss D2H),
metrics and checkpoint/resume. One process drives one GPU.
"""
from __future__ import annotations

import json
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .config import LlamaConfig, MeshConfig, TrainConfig
from .models.llama import LlamaModel, StepContext
from .models.params import FlatParams
from .ops import _lib
from .ops import kernels as K
from .ops.reference import balanced_pairs, shard_positions
from .parallel import gradsync
from .parallel.mesh import DeviceMesh
from .utils.tracing import phase


def init_distributed(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """Initialise ``torch.distributed`` from the torchrun environment (no-op for one process).
    Returns ``(rank, world_size, local_rank)``."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        be = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        kwargs = {}
        if be == "nccl":
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=be, rank=rank, world_size=world, **kwargs)
    return rank, world, local


def geometric_segment_ids(batch: int, seq_len: int, mean_len: int, generator: torch.Generator) -> torch.Tensor:
    """Packed documents: lengths ~ Geometric(1/mean_len), truncated to the sequence; returns
    ``(batch, seq_len)`` int32 ids that increase along the sequence."""
    p = 1.0 / float(mean_len)
    boundary = torch.rand(batch, seq_len, generator=generator) < p
    boundary[:, 0] = False
    return torch.cumsum(boundary.to(torch.int32), dim=1).to(torch.int32)


def synthetic_batch(cfg: LlamaConfig, batch: int, seq_len: int, generator: torch.Generator,
                    mean_doc_len: int = 0):
    """Uniform random tokens in ``[0, vocab)`` with next-token targets (the last position, and the
    last token of every packed document, has target -1). CPU tensors."""
    tokens = torch.randint(0, cfg.vocab_size, (batch, seq_len), generator=generator, dtype=torch.int32)
    targets = torch.full_like(tokens, -1)
    targets[:, :-1] = tokens[:, 1:]
    seg = None
    if mean_doc_len > 0:
        seg = geometric_segment_ids(batch, seq_len, mean_doc_len, generator)
        last = torch.ones_like(seg, dtype=torch.bool)
        last[:, :-1] = seg[:, 1:] != seg[:, :-1]
        targets[last] = -1
    return tokens, targets, seg


class PeerLost(RuntimeError):
    """Another rank announced that it left the job; nothing was launched for this step."""


class Trainer:
    """Owns the model replica of this rank and runs training steps on the mesh.

    Mesh semantics: ``sp`` shards the sequence (ring attention), ``dp`` and ``fsdp`` shard the
    batch; the bf16 parameters are replicated over ``sp``/``dp``; over ``fsdp`` every GEMM weight, its fp32
    master copy and its AdamW moments are row-sharded, and the shards of the other ranks are pulled
    inside the GEMM that needs them (see ``models/params.py``). With ``TrainConfig.zero1`` (the default) the
    fp32 master weights and the AdamW moments are also cut into equal slices over the sp/dp ranks that
    hold the same parameters: gradients are reduce-scattered, each rank updates its slice, and the bf16
    weights are all-gathered (``parallel/gradsync.py``).
    """

    def __init__(self, model_cfg: LlamaConfig, train_cfg: TrainConfig, mesh: Optional[DeviceMesh] = None,
                 device: Optional[torch.device] = None, standalone: bool = False):
        self.cfg = model_cfg
        self.tc = train_cfg
        tp = mesh.size("tp") if mesh is not None else MeshConfig.parse(train_cfg.mesh).tp
        if tp != 1:
            # the tp axis exists so that (dp, fsdp, tp, sp) specs can be written down; the driver model has no
            # tensor-parallel layers, and tp ranks would be replicas on the same data counted tp times
            raise ValueError("tensor parallelism is not implemented in this driver: the mesh must have tp = 1")
        self.rank, self.world, self.local_rank = init_distributed()
        if standalone:  # a one-rank replica inside a larger job: joins no collective
            self.rank, self.world = 0, 1
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.mesh = mesh or DeviceMesh(MeshConfig.parse(train_cfg.mesh), register=not standalone,
                                       standalone=standalone)
        self.sp_rank, self.sp = self.mesh.index("sp"), self.mesh.size("sp")
        self.fsdp_rank, self.fsdp = self.mesh.index("fsdp"), self.mesh.size("fsdp")
        self.dp_rank, self.dp = self.mesh.index("dp"), self.mesh.size("dp")
        self.batch_groups = self.dp * self.fsdp
        self.batch_index = self.dp_rank * self.fsdp + self.fsdp_rank
        if train_cfg.global_batch % self.batch_groups:
            raise ValueError("global_batch must be divisible by dp*fsdp")
        if train_cfg.seq_len % self.sp:
            raise ValueError("seq_len must be divisible by sp")
        self.B = train_cfg.global_batch // self.batch_groups
        self.S = train_cfg.seq_len // self.sp
        # ranks that hold the same parameter shard (same fsdp coordinate): they reduce its gradient together,
        # and (train_cfg.zero1) each keeps one slice of its optimizer state
        self._replica_group = None
        if self.world > 1 and not standalone:
            self._replica_group = self.mesh.replica_group("fsdp") if self.fsdp > 1 else dist.group.WORLD
        self.zero = None
        if train_cfg.zero1 and self._replica_group is not None and dist.get_world_size(self._replica_group) > 1:
            self.zero = (dist.get_rank(self._replica_group), dist.get_world_size(self._replica_group),
                         self._replica_group)
        params = FlatParams(model_cfg, self.device, seed=train_cfg.seed, with_optimizer=True,
                            shard=(self.fsdp_rank, self.fsdp),
                            fsdp_group=self.mesh.axis("fsdp").group if self.fsdp > 1 else None, zero=self.zero)
        self.model = LlamaModel(model_cfg, self.device, params=params)
        self.symm_ring = None
        if self.sp > 1:
            from .parallel.symm import SymmRing

            self.symm_ring = SymmRing(self.mesh.axis("sp").group, self.device)
            self.mesh.axis("sp").symm_ring = self.symm_ring
        self.step_idx = 0
        self._sync_token = torch.zeros(1, device=self.device)
        self.gnorm_sq = torch.zeros(1, device=self.device, dtype=torch.float32)
        self.gen = torch.Generator()
        self.gen.manual_seed(train_cfg.seed + 1)
        # pinned staging for the per-step host->device input copy
        n = self.B * self.S
        self._tok_host = torch.empty(self.B, self.S, dtype=torch.int32).pin_memory()
        self._tgt_host = torch.empty(self.B, self.S, dtype=torch.int32).pin_memory()
        self._tok_dev = torch.empty(self.B, self.S, dtype=torch.int32, device=self.device)
        self._tgt_dev = torch.empty(self.B, self.S, dtype=torch.int32, device=self.device)
        self._loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self._ctx_cache: Optional[StepContext] = None
        self._ctx_seg_key = None
        self._layout, self._layout_key = None, None

    # ------------------------------------------------------------------ data
    def make_global_batch(self):
        """Synthetic global batch (identical on every rank: same generator seed)."""
        return synthetic_batch(self.cfg, self.tc.global_batch, self.tc.seq_len, self.gen,
                               self.tc.packed_mean_doc_len)

    def layout_for(self, segment_ids=None) -> str:
        """Token layout of the ring for a batch: the configured one, or, for packed documents on a two-run layout
        (``TrainConfig.balance_documents``), the pairing of half-chunks that balances the documents' attention work
        over the ranks of this ring (``ops.reference.balanced_pairs``). All ranks of a ring see the same rows and
        get the same answer."""
        if segment_ids is None or self.sp == 1 or self.cfg.layout == "contiguous" or not self.tc.balance_documents:
            return self.cfg.layout
        key = (segment_ids.data_ptr(), tuple(segment_ids.shape), segment_ids._version)
        if self._layout_key != key:
            b0 = self.batch_index * self.B
            self._layout, self._layout_key = balanced_pairs(segment_ids[b0:b0 + self.B], self.sp), key
        return self._layout

    def shard_batch(self, tokens, targets, segment_ids=None):
        """Slice this rank's rows (batch groups) and token positions (sp shard, layout-aware)."""
        b0 = self.batch_index * self.B
        pos = shard_positions(self.sp_rank, self.sp, self.S, self.layout_for(segment_ids))
        return (tokens[b0:b0 + self.B].index_select(1, pos), targets[b0:b0 + self.B].index_select(1, pos))

    def h2d_bytes_per_step(self) -> int:
        return self._tok_host.numel() * 4 + self._tgt_host.numel() * 4

    def d2h_bytes_per_step(self) -> int:
        return 4

    # ------------------------------------------------------------------ step
    def context(self, segment_ids=None) -> StepContext:
        key = None if segment_ids is None else (segment_ids.data_ptr(), tuple(segment_ids.shape),
                                                segment_ids._version)
        if self._ctx_cache is None or key != self._ctx_seg_key:
            b0 = self.batch_index * self.B
            seg = None if segment_ids is None else segment_ids[b0:b0 + self.B].to(self.device)
            self._attn_pairs = None
            if segment_ids is not None:
                # visible (q, k) pairs of the whole global batch, for the FLOP count: same document, k <= q
                flat = segment_ids.long() + torch.arange(segment_ids.shape[0])[:, None] * (int(segment_ids.max()) + 1)
                ln = torch.bincount(flat.flatten()).double()
                self._attn_pairs = float((ln * (ln + 1) / 2).sum())
            self._ctx_cache = self.model.make_context(
                self.B, self.S, self.sp_rank, self.sp, segment_ids=seg, symm_ring=self.symm_ring,
                total_tokens=self.tc.global_batch * self.tc.seq_len, layout=self.layout_for(segment_ids))
            self._ctx_seg_key = key
        return self._ctx_cache

    def device_step(self, tok_dev, tgt_dev, ctx: StepContext) -> torch.Tensor:
        """Forward/backward, gradient reduction and optimizer update on device-resident inputs.
        Returns the global mean loss as a 0-d device tensor."""
        P = self.model.params
        with phase("step_total"):
            P.ensure_grads().zero_()
            loss_sum = self.model.forward_backward(tok_dev, tgt_dev, ctx)
            if self.world > 1:
                with phase("grad_allreduce"):
                    dist.all_reduce(loss_sum)
                    self._all_reduce_grads()
            with phase("optimizer"):
                self.optimizer_step()
        return loss_sum / max(1, ctx.total_tokens)

    def _all_reduce_grads(self, bucket: int = 1 << 28) -> None:
        """Sum the gradients over the job: all-reduce, or with fsdp > 1 a reduce-scatter over the fsdp
        axis plus an all-reduce of the owned shard over the ranks sharing the fsdp coordinate."""
        P = self.model.params
        fsdp_group = self.mesh.axis("fsdp").group if self.fsdp > 1 else None
        if self.zero is not None:
            gradsync.reduce_gradients_zero(P.g32, P.numel_shard, P.shard_count, P.shard_index, fsdp_group, self.zero)
            return
        gradsync.reduce_gradients(P.g32, P.numel_shard, P.shard_count, P.shard_index, fsdp_group,
                                  self._replica_group if self.fsdp > 1 else None, bucket)

    def optimizer_step(self) -> None:
        P, tc = self.model.params, self.tc
        self.step_idx += 1
        clip = float(tc.grad_clip)
        if clip > 0:
            self.gnorm_sq.zero_()
            if self.zero is not None:  # only the owned slices hold full sums
                tail = torch.zeros_like(self.gnorm_sq)
                K.sumsq(P.own(P.grad_shard(P.shard_index)), self.gnorm_sq)
                K.sumsq(P.own(P.grad_rep()), tail)
                self.gnorm_sq.copy_(gradsync.global_sumsq_zero(
                    self.gnorm_sq, tail, self.mesh.axis("fsdp").group if self.fsdp > 1 else None, self.zero))
            elif self.fsdp == 1:
                K.sumsq(P.g32, self.gnorm_sq)
            else:  # only the owned shard and the replicated tail hold full sums
                tail = torch.zeros_like(self.gnorm_sq)
                K.sumsq(P.grad_shard(P.shard_index), self.gnorm_sq)
                K.sumsq(P.grad_rep(), tail)
                self.gnorm_sq.copy_(gradsync.global_sumsq(self.gnorm_sq, tail, self.mesh.axis("fsdp").group))
        P.adamw_step(self.step_idx, tc.lr, tc.beta1, tc.beta2, tc.eps, tc.weight_decay, clip,
                     self.gnorm_sq if clip > 0 else None)
        if self.fsdp > 1:
            # peers pull this rank's shard inside their GEMMs: order the update before their next step
            dist.all_reduce(self._sync_token, group=self.mesh.axis("fsdp").group)

    # ------------------------------------------------------------------ failure detection (host side)
    def _store(self):
        if self.world == 1:
            return None
        from torch.distributed import distributed_c10d as c10d

        return c10d._get_default_store()

    def leave(self) -> None:
        """Announce that this rank stops taking part (call between steps, nothing in flight)."""
        torch.cuda.synchronize(self.device)
        st = self._store()
        if st is not None:
            st.add("ringattn_b200/left", 1)

    def check_peers(self) -> None:
        """Raise :class:`PeerLost` before launching anything if a peer has left. Kernels that touch
        peer memory are only launched after this check; a peer that dies without announcing it is
        caught by the bounded ring barrier (status word) or the process-group timeout."""
        st = self._store()
        if st is not None and st.add("ringattn_b200/left", 0) > 0:
            raise PeerLost(f"rank {self.rank}: a peer left the job; step {self.step_idx + 1} not launched")

    def train_step(self, tokens_cpu, targets_cpu, segment_ids=None) -> float:
        """The end-to-end step a user calls: sharded inputs come from pinned host memory, the loss
        comes back to the host."""
        self.check_peers()
        tok, tgt = self.shard_batch(tokens_cpu, targets_cpu, segment_ids)
        self._tok_host.copy_(tok)
        self._tgt_host.copy_(tgt)
        self._tok_dev.copy_(self._tok_host, non_blocking=True)
        self._tgt_dev.copy_(self._tgt_host, non_blocking=True)
        ctx = self.context(segment_ids)
        loss = self.device_step(self._tok_dev, self._tgt_dev, ctx)
        self._loss_host.copy_(loss.reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        _lib.check_status(self.device)
        return float(self._loss_host[0])

    # ------------------------------------------------------------------ metrics
    def model_flops_per_step(self) -> float:
        """Model FLOPs of one step (forward + backward, no recomputation): 6 per matmul parameter and
        token, plus 12 * d_model per layer and visible (query, key) pair. With packed documents only
        pairs inside a document count."""
        tokens = self.tc.global_batch * self.tc.seq_len
        dense = self.model.flops_per_token(0) * tokens
        pairs = getattr(self, "_attn_pairs", None)
        if pairs is None:
            pairs = self.tc.global_batch * self.tc.seq_len * (self.tc.seq_len + 1) / 2.0
        return dense + 12.0 * self.cfg.n_layers * self.cfg.d_model * pairs

    # ------------------------------------------------------------------ checkpoint / resume
    def save_checkpoint(self, directory: str) -> str:
        """Each rank writes its optimizer shard; rank 0 of every parameter replica set also writes
        the metadata. Files: ``rank{r}.pt`` and ``meta.json``."""
        os.makedirs(directory, exist_ok=True)
        P = self.model.params
        path = os.path.join(directory, f"rank{self.rank}.pt")
        st = P.state_dict()
        st.update(step=self.step_idx, gen=self.gen.get_state())
        torch.save(st, path)
        if self.rank == 0:
            with open(os.path.join(directory, "meta.json"), "w") as f:
                json.dump({"step": self.step_idx, "world": self.world, "mesh": self.mesh.config.shape(),
                           "model": self.cfg.__dict__, "train": self.tc.asdict()}, f, default=str)
        if self.world > 1:
            dist.barrier()
        return path

    def load_checkpoint(self, directory: str) -> None:
        st = torch.load(os.path.join(directory, f"rank{self.rank}.pt"), map_location="cpu")
        self.model.params.load_state_dict(st)
        self.step_idx = int(st["step"])
        self.gen.set_state(st["gen"])
        if self.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier()
