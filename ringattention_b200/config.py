"""Configuration objects: ``BlockwiseKwargs`` (the reference's ``blockwise_kwargs`` dict, validated),
``MeshConfig`` (dp, fsdp, tp, sp), ``LlamaConfig`` and ``TrainConfig``.

The reference has no config system: it passes a plain dict whose ten keys are positional
parameters of its blockwise functions (ringattention/ringattention_jax.py:99-100, README.md:25-36).
``BlockwiseKwargs.from_any`` accepts that dict verbatim.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch

# Remat policies understood by this library. The reference forwards a jax.checkpoint policy
# (ringattention_jax.py:130,334); only the two below have an effect here.
POLICY_NOTHING_SAVEABLE = "nothing_saveable"
POLICY_EVERYTHING_SAVEABLE = "everything_saveable"
# Model-level extension: recompute a layer in the backward pass except its attention, whose output and
# log-sum-exp are kept (0.5 GB per layer at 64K tokens x 4096). Not one of the reference's policies.
POLICY_SAVE_ATTENTION = "save_attention"

_REFERENCE_KEYS = (
    "causal_block_size", "query_chunk_size", "key_chunk_size", "deterministic", "dropout_rng",
    "attn_pdrop", "dtype", "policy", "precision", "prevent_cse",
)
_EXTENSION_KEYS = ("layout",)


def _policy_name(policy: Any) -> str:
    if policy is None:
        return POLICY_NOTHING_SAVEABLE
    if isinstance(policy, str):
        name = policy
    else:  # e.g. a function object named like jax.checkpoint_policies.nothing_saveable
        name = getattr(policy, "__name__", str(policy))
    if "nothing" in name:
        return POLICY_NOTHING_SAVEABLE
    if "everything" in name or "dots" in name or "save" in name:
        return POLICY_EVERYTHING_SAVEABLE
    raise ValueError(f"unknown remat policy {policy!r}")


@dataclass
class BlockwiseKwargs:
    """Validated form of the reference's ``blockwise_kwargs``.

    ``causal_block_size``: ``None`` no causal mask, 1 causal, k>1 block-causal (token i sees j iff
    ``i // k >= j // k``; ringattention_jax.py:301-309). ``query_chunk_size``/``key_chunk_size`` must
    divide the local lengths (ringattention_jax.py:104-108); results do not depend on them.
    Dropout is active iff ``not deterministic and attn_pdrop > 0``; dropped logits are masked before
    the softmax without 1/(1-p) rescaling (ringattention_jax.py:119-123,311-321).
    ``dropout_rng`` is an int seed or a ``torch.Generator`` (a seed is drawn from it).
    ``layout`` is an extension: ``"contiguous"`` (reference behaviour: rank r owns tokens
    ``[r*c, (r+1)*c)``), ``"zigzag"`` (rank r owns chunks r and 2N-1-r of 2N, which balances
    causal work across the ring) or ``"pairs:a0-b0,..."`` (an explicit pairing of the 2N half-chunks, e.g. the one
    ``ops.reference.balanced_pairs`` derives from the document boundaries of a packed batch).
    """

    causal_block_size: Optional[int] = None
    query_chunk_size: int = 128
    key_chunk_size: int = 128
    deterministic: bool = True
    dropout_rng: Any = None
    attn_pdrop: float = 0.0
    dtype: Any = torch.float32
    policy: str = POLICY_NOTHING_SAVEABLE
    precision: Any = None
    prevent_cse: bool = True
    layout: str = "contiguous"

    @classmethod
    def from_any(cls, obj: "BlockwiseKwargs | Mapping[str, Any] | None") -> "BlockwiseKwargs":
        if obj is None:
            return cls()
        if isinstance(obj, cls):
            return obj
        if not isinstance(obj, Mapping):
            raise TypeError("blockwise_kwargs must be a dict or BlockwiseKwargs")
        unknown = set(obj) - set(_REFERENCE_KEYS) - set(_EXTENSION_KEYS)
        if unknown:
            raise KeyError(f"unknown blockwise_kwargs keys: {sorted(unknown)}")
        kw = dict(obj)
        if "policy" in kw:
            kw["policy"] = _policy_name(kw["policy"])
        out = cls(**kw)
        out.validate()
        return out

    def validate(self) -> None:
        if self.causal_block_size is not None and int(self.causal_block_size) < 1:
            raise ValueError("causal_block_size must be None or >= 1")
        if self.query_chunk_size < 1 or self.key_chunk_size < 1:
            raise ValueError("chunk sizes must be positive")
        if not (0.0 <= float(self.attn_pdrop) < 1.0):
            raise ValueError("attn_pdrop must be in [0, 1)")
        if self.layout not in ("contiguous", "zigzag") and not str(self.layout).startswith("pairs:"):
            raise ValueError("layout must be 'contiguous', 'zigzag' or 'pairs:a0-b0,a1-b1,...'")

    @property
    def dropout_active(self) -> bool:
        return (not self.deterministic) and float(self.attn_pdrop) > 0.0

    def seed(self) -> int:
        """64-bit dropout seed derived from ``dropout_rng`` (0 when dropout is inactive)."""
        if not self.dropout_active:
            return 0
        rng = self.dropout_rng
        if rng is None:
            raise ValueError("dropout is active but dropout_rng is None")
        if isinstance(rng, torch.Generator):
            return int(torch.randint(0, 2**62, (1,), generator=rng).item())
        if isinstance(rng, torch.Tensor):
            return int(rng.flatten()[0].item()) & (2**63 - 1)
        return int(rng) & (2**63 - 1)


@dataclass(frozen=True)
class SegmentIds:
    """Per-token segment ids of the queries and of the keys/values of one attention call (the
    reference's ``SegmentIds`` NamedTuple, ringattention_pallas_tpu.py:201-215). Tokens attend only
    to tokens with an equal id."""

    q: Any
    kv: Any


@dataclass(frozen=True)
class BlockSizes:
    """Tile sizes of the fused kernels. The reference exposes eleven tunable TPU tile sizes
    (ringattention_pallas_tpu.py:218-287, default 128 everywhere); the sm_100a kernels are built for
    one tile shape, fixed by the tcgen05 instruction shape and the TMEM budget, so this object is
    informational: ``validate`` only checks that a request is compatible."""

    block_q: int = 256          # query rows per CTA in the forward (two 128-row tiles)
    block_k: int = 128          # key rows per pipeline step
    block_q_bwd: int = 128      # query rows per backward iteration
    block_k_bwd: int = 128      # key rows per backward CTA
    block_b: int = 1

    @classmethod
    def get_default(cls) -> "BlockSizes":
        return cls()

    def validate(self, q_len: int, kv_len: int) -> None:
        if self.block_b != 1:
            raise ValueError("block_b must be 1")
        for name in ("block_q", "block_k", "block_q_bwd", "block_k_bwd"):
            v = getattr(self, name)
            if v % 128:
                raise ValueError(f"{name} must be a multiple of 128")
        if q_len < 1 or kv_len < 1:
            raise ValueError("empty sequence")


@dataclass
class MeshConfig:
    """Sizes of the four mesh axes used in the reference's README (README.md:38-46)."""

    dp: int = 1
    fsdp: int = 1
    tp: int = 1
    sp: int = 1

    AXES = ("dp", "fsdp", "tp", "sp")

    @classmethod
    def parse(cls, text: "str | MeshConfig | None") -> "MeshConfig":
        """Parse ``"1,2,1,4"`` (dp,fsdp,tp,sp) or ``"fsdp=2,sp=4"``."""
        if text is None:
            return cls()
        if isinstance(text, cls):
            return text
        parts = [p.strip() for p in str(text).split(",") if p.strip()]
        if all("=" in p for p in parts):
            kv = {}
            for p in parts:
                k, v = p.split("=")
                if k.strip() not in cls.AXES:
                    raise ValueError(f"unknown mesh axis {k!r}")
                kv[k.strip()] = int(v)
            return cls(**kv)
        if len(parts) != 4:
            raise ValueError("mesh must be 'dp,fsdp,tp,sp' or 'axis=size,...'")
        return cls(*[int(p) for p in parts])

    @property
    def world_size(self) -> int:
        return self.dp * self.fsdp * self.tp * self.sp

    def shape(self) -> tuple[int, int, int, int]:
        return (self.dp, self.fsdp, self.tp, self.sp)

    def describe(self) -> str:
        return "x".join(f"{a}{getattr(self, a)}" for a in self.AXES if getattr(self, a) > 1) or "single"


@dataclass
class LlamaConfig:
    """LLaMA-style decoder. Defaults are the 7B shape."""

    vocab_size: int = 32000
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    d_ff: int = 11008
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0
    init_std: float = 0.02
    max_seq_len: int = 1 << 20
    # attention / ffn chunking
    query_chunk_size: int = 2048
    key_chunk_size: int = 2048
    ffn_chunk_size: int = 8192
    loss_chunk_size: int = 8192
    causal_block_size: int = 1
    remat: str = POLICY_NOTHING_SAVEABLE
    layout: str = "contiguous"

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def n_params(self, include_embedding: bool = True) -> int:
        per_layer = 4 * self.d_model * self.d_model + 3 * self.d_model * self.d_ff + 2 * self.d_model
        n = self.n_layers * per_layer + self.d_model + self.vocab_size * self.d_model
        if include_embedding:
            n += self.vocab_size * self.d_model
        return n

    @classmethod
    def named(cls, name: str, **over) -> "LlamaConfig":
        presets = {
            "llama-7b": dict(),
            "llama-1b": dict(d_model=2048, n_layers=16, n_heads=16, d_ff=5504),
            "llama-tiny": dict(vocab_size=1024, d_model=256, n_layers=2, n_heads=2, d_ff=512,
                               query_chunk_size=128, key_chunk_size=128, ffn_chunk_size=256,
                               loss_chunk_size=256),
            "llama-small": dict(vocab_size=4096, d_model=512, n_layers=2, n_heads=4, d_ff=1536,
                                query_chunk_size=256, key_chunk_size=256, ffn_chunk_size=512,
                                loss_chunk_size=512),
        }
        if name not in presets:
            raise KeyError(f"unknown model {name!r}; have {sorted(presets)}")
        kw = dict(presets[name])
        kw.update(over)
        return cls(**kw)


@dataclass
class TrainConfig:
    model: str = "llama-7b"
    mesh: str = "1,1,1,1"
    seq_len: int = 65536          # global sequence length
    global_batch: int = 1
    lr: float = 1e-4
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    grad_clip: float = 1.0
    steps: int = 10
    seed: int = 0
    packed_mean_doc_len: int = 0  # >0: packed documents with geometric lengths (segment ids)
    balance_documents: bool = True  # packed documents on a ring: pair the half-chunks by their attention work
    zero1: bool = True            # shard fp32 master weights and AdamW moments over the sp/dp replicas
    log_every: int = 1
    ckpt_dir: Optional[str] = None
    ckpt_every: int = 0
    resume: bool = False

    def asdict(self) -> dict:
        return dataclasses.asdict(self)
