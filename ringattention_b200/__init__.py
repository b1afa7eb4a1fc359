"""ringattention_b200: ring attention and a LLaMA training/inference driver written for B200
(sm_100a): tcgen05/TMEM/TMA kernels, KV blocks pulled over NVLink from inside the attention
kernels, one process per GPU.

Public names (the reference exports ``ringattention``, ``blockwise_feedforward``,
``ringattention_jax`` and ``ringattention_inference``, ringattention/__init__.py:26-27):
"""
from .api import blockwise_feedforward, ringattention, ringattention_inference, ringattention_ref
from .config import BlockSizes, BlockwiseKwargs, LlamaConfig, MeshConfig, SegmentIds, TrainConfig

# the reference's name for its pure-framework implementation
ringattention_jax = ringattention_ref

__all__ = [
    "ringattention", "blockwise_feedforward", "ringattention_inference", "ringattention_ref",
    "ringattention_jax", "BlockwiseKwargs", "BlockSizes", "SegmentIds", "LlamaConfig", "MeshConfig", "TrainConfig",
]
__version__ = "0.1.0"
