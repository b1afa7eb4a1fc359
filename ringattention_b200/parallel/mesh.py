"""The ``(dp, fsdp, tp, sp)`` device mesh and the axis-name registry.

The reference is called inside ``shard_map`` over a mesh with these four axes and finds its ring
through ``axis_name`` (README.md:19-49; ringattention_jax.py:24,32,47). Here one process drives one
GPU; :class:`DeviceMesh` maps the global rank to mesh coordinates (``sp`` varies fastest, so the
ranks of one ring are neighbours on the NVSwitch fabric), builds one ``torch.distributed`` group per
axis and registers an :class:`AxisContext` under each axis name. ``ringattention(...,
axis_name="sp")`` looks the ring up in that registry.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..config import MeshConfig
from .comm import RingComm, SingleComm, TorchDistRing


@dataclass
class AxisContext:
    """What an axis name resolves to: a rotation communicator (CPU path / baseline) and, on GPUs,
    the symmetric-memory ring used by the fused kernels."""

    name: str
    comm: RingComm
    group: Optional[Any] = None
    symm_ring: Optional[Any] = None  # parallel.symm.SymmRing, created lazily on CUDA

    @property
    def rank(self) -> int:
        return self.comm.rank

    @property
    def size(self) -> int:
        return self.comm.size


_GLOBAL_AXES: Dict[str, AxisContext] = {}
_LOCAL = threading.local()


def register_axis(name: str, comm: RingComm, group=None, thread_local: bool = False) -> AxisContext:
    """Bind ``name`` to a communicator. ``thread_local=True`` is for in-process fake rings, where
    every thread plays a different rank."""
    ctx = AxisContext(name=name, comm=comm, group=group)
    if thread_local:
        if not hasattr(_LOCAL, "axes"):
            _LOCAL.axes = {}
        _LOCAL.axes[name] = ctx
    else:
        _GLOBAL_AXES[name] = ctx
    return ctx


def unregister_axis(name: str) -> None:
    _GLOBAL_AXES.pop(name, None)
    if hasattr(_LOCAL, "axes"):
        _LOCAL.axes.pop(name, None)


def resolve_axis(axis: "str | RingComm | AxisContext | None") -> AxisContext:
    """Axis name / communicator / ``None`` -> :class:`AxisContext` (``None`` = single device)."""
    if axis is None:
        return AxisContext(name="", comm=SingleComm())
    if isinstance(axis, AxisContext):
        return axis
    if isinstance(axis, RingComm):
        return AxisContext(name="", comm=axis)
    if isinstance(axis, str):
        local = getattr(_LOCAL, "axes", {})
        if axis in local:
            return local[axis]
        if axis in _GLOBAL_AXES:
            return _GLOBAL_AXES[axis]
        raise KeyError(f"axis {axis!r} is not registered; create a DeviceMesh or call register_axis")
    raise TypeError(f"cannot resolve axis from {type(axis).__name__}")


class DeviceMesh:
    """Mesh over the ranks of the default process group. ``coords`` are this rank's
    ``(dp, fsdp, tp, sp)`` indices; ``axis(name)`` returns the registered :class:`AxisContext`."""

    AXES = MeshConfig.AXES

    def __init__(self, config: "MeshConfig | str", register: bool = True, standalone: bool = False):
        """``standalone=True`` builds a one-rank mesh even inside a multi-process job (a replica that
        takes no part in any collective; used for single-device reference runs)."""
        self.config = MeshConfig.parse(config)
        if not standalone and dist.is_available() and dist.is_initialized():
            self.world_size = dist.get_world_size()
            self.rank = dist.get_rank()
        else:
            self.world_size, self.rank = 1, 0
        if self.config.world_size != self.world_size:
            raise ValueError(f"mesh {self.config.shape()} needs {self.config.world_size} ranks, "
                             f"world size is {self.world_size}")
        self.coords = self.rank_to_coords(self.rank)
        self._axes: Dict[str, AxisContext] = {}
        for ai, name in enumerate(self.AXES):
            size = self.config.shape()[ai]
            if self.world_size == 1 or size == 1:
                ctx = AxisContext(name=name, comm=SingleComm())
            else:
                ctx = self._make_axis_group(ai, name)
            self._axes[name] = ctx
            if register:
                _GLOBAL_AXES[name] = ctx

    # rank = ((dp * FSDP + fsdp) * TP + tp) * SP + sp
    def rank_to_coords(self, rank: int) -> tuple:
        dp, fs, tp, sp = self.config.shape()
        c_sp = rank % sp
        c_tp = (rank // sp) % tp
        c_fs = (rank // (sp * tp)) % fs
        c_dp = rank // (sp * tp * fs)
        return (c_dp, c_fs, c_tp, c_sp)

    def coords_to_rank(self, coords) -> int:
        dp, fs, tp, sp = self.config.shape()
        return ((coords[0] * fs + coords[1]) * tp + coords[2]) * sp + coords[3]

    def _make_axis_group(self, axis_index: int, name: str) -> AxisContext:
        shape = self.config.shape()
        my_group = None
        # every rank must create every group, in the same order
        others = [i for i in range(4) if i != axis_index]
        import itertools

        for fixed in itertools.product(*[range(shape[i]) for i in others]):
            ranks = []
            for v in range(shape[axis_index]):
                c = [0, 0, 0, 0]
                for i, f in zip(others, fixed):
                    c[i] = f
                c[axis_index] = v
                ranks.append(self.coords_to_rank(c))
            g = dist.new_group(ranks)
            if self.rank in ranks:
                my_group = g
        return AxisContext(name=name, comm=TorchDistRing(my_group), group=my_group)

    def axis(self, name: str) -> AxisContext:
        return self._axes[name]

    def replica_group(self, name: str):
        """Process group of the ranks that share this rank's coordinate on axis ``name`` (every
        combination of the other axes); ``None`` when that is this rank alone or there is no process
        group. Collective: every rank of the job must call it, in the same order."""
        if self.world_size == 1 or self.size(name) == self.world_size:
            return None
        ai = self.AXES.index(name)
        mine = None
        for v in range(self.config.shape()[ai]):
            ranks = [r for r in range(self.world_size) if self.rank_to_coords(r)[ai] == v]
            g = dist.new_group(ranks)
            if self.coords[ai] == v:
                mine = g
        return mine

    def size(self, name: str) -> int:
        return self._axes[name].size

    def index(self, name: str) -> int:
        return self.coords[self.AXES.index(name)]

    def describe(self) -> str:
        return self.config.describe()
