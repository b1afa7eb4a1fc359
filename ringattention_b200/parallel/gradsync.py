"""Gradient reduction for the ``(dp, fsdp, tp, sp)`` mesh.

Every rank computes the gradient of *all* parameters on its own tokens: a flat fp32 buffer laid out
``[shard 0 | shard 1 | ... | shard f-1 | replicated]`` (shard s = the rows that fsdp rank s owns). The
optimizer of a rank only touches its own shard and the replicated tail, so the reduction is a
reduce-scatter over the ``fsdp`` axis followed by an all-reduce of the owned shard over the ranks that
share the fsdp coordinate, instead of an all-reduce of everything: ``(f-1)/f + 2/f`` buffer volumes
per rank instead of 2. With ``f == 1`` it degenerates to the plain all-reduce.

The reduce-scatter is issued as one ``reduce`` per shard (root = the owner), which exists on every
backend (NCCL, gloo), in buckets so that no single collective exceeds ``bucket`` elements.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _bucketed(fn, t: torch.Tensor, bucket: int) -> None:
    for s0 in range(0, t.numel(), bucket):
        fn(t[s0:s0 + bucket])


def reduce_gradients(g: torch.Tensor, numel_shard: int, n_shards: int, my_shard: int,
                     fsdp_group=None, replica_group=None, bucket: int = 1 << 28) -> None:
    """In place. Afterwards ``g[my_shard * numel_shard : (my_shard + 1) * numel_shard]`` and the
    replicated tail hold the sums over all ranks; the other shards' segments are left in an
    unspecified state (partial sums) and must not be used.

    ``fsdp_group``: the ranks that differ only in the fsdp coordinate (None when ``n_shards == 1``).
    ``replica_group``: the ranks that share this rank's fsdp coordinate (all dp/tp/sp combinations);
    None means "nobody else" (world == fsdp group)."""
    if not (dist.is_available() and dist.is_initialized()):
        return
    tail = g[n_shards * numel_shard:]
    if n_shards == 1:
        _bucketed(lambda x: dist.all_reduce(x), g, bucket)
        return
    for s in range(n_shards):
        root = dist.get_global_rank(fsdp_group, s)
        seg = g[s * numel_shard:(s + 1) * numel_shard]
        _bucketed(lambda x: dist.reduce(x, dst=root, group=fsdp_group), seg, bucket)
    if replica_group is not None and dist.get_world_size(replica_group) > 1:
        mine = g[my_shard * numel_shard:(my_shard + 1) * numel_shard]
        _bucketed(lambda x: dist.all_reduce(x, group=replica_group), mine, bucket)
    if tail.numel():
        _bucketed(lambda x: dist.all_reduce(x), tail, bucket)


def global_sumsq(own_sq: torch.Tensor, tail_sq: torch.Tensor, fsdp_group=None) -> torch.Tensor:
    """Squared gradient norm of the whole model from the squared norm of the owned shard (summed over
    the fsdp group: the shards are disjoint) and of the replicated tail (identical on all ranks)."""
    total = own_sq.clone()
    if fsdp_group is not None and dist.get_world_size(fsdp_group) > 1:
        dist.all_reduce(total, group=fsdp_group)
    return total + tail_sq
