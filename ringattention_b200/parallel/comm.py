"""Ring communicators for the *rotation* form of ring attention (CPU path and NCCL baseline).

The reference moves K/V (and dK/dV) one hop per ring step with ``lax.ppermute``
(ringattention/ringattention_jax.py:47,85-86). ``RingComm.send_recv`` is that hop: every rank sends
its tensors to ``rank+1`` and receives the ones of ``rank-1``.

* :class:`SingleComm` - one rank, no traffic.
* :class:`TorchDistRing` - ``torch.distributed`` ``batch_isend_irecv`` over gloo (CPU tests) or NCCL
  (the GPU *baseline*; the product path pulls KV from peer memory inside the attention kernel
  instead, see :mod:`ringattention_b200.parallel.symm`).
* :class:`FakeRing` - N ranks as threads of one process connected by queues, for fast unit tests.
  A rank can be told to drop out or to lose a message, which is how failure handling is tested
  without touching a GPU.
"""
from __future__ import annotations

import queue
import threading
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


class RingTimeout(RuntimeError):
    """A peer did not deliver within the deadline."""


class RingComm:
    rank: int = 0
    size: int = 1

    def send_recv(self, tensors: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        raise NotImplementedError

    def barrier(self) -> None:
        pass

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        return t


class SingleComm(RingComm):
    def send_recv(self, tensors):
        return list(tensors)


class TorchDistRing(RingComm):
    """Ring over a ``torch.distributed`` process group (gloo or nccl)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self._next = dist.get_global_rank(group, (self.rank + 1) % self.size) if group is not None \
            else (self.rank + 1) % self.size
        self._prev = dist.get_global_rank(group, (self.rank - 1) % self.size) if group is not None \
            else (self.rank - 1) % self.size

    def send_recv(self, tensors):
        if self.size == 1:
            return list(tensors)
        sends = [t.contiguous() for t in tensors]
        recvs = [torch.empty_like(t) for t in sends]
        ops = []
        for s, r in zip(sends, recvs):
            ops.append(dist.P2POp(dist.isend, s, self._next, group=self.group))
            ops.append(dist.P2POp(dist.irecv, r, self._prev, group=self.group))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        return recvs

    def barrier(self):
        dist.barrier(group=self.group)

    def all_reduce_sum(self, t):
        dist.all_reduce(t, group=self.group)
        return t


class _FakeRingShared:
    def __init__(self, size: int, timeout: float):
        self.size = size
        self.timeout = timeout
        self.queues = [queue.Queue() for _ in range(size)]  # inbox of rank i (from rank i-1)
        self.barrier = threading.Barrier(size)
        self.drop_next_message_to: set[int] = set()
        self.lock = threading.Lock()


class FakeRing(RingComm):
    """One endpoint of an in-process ring; create all endpoints with :meth:`create`."""

    def __init__(self, shared: _FakeRingShared, rank: int):
        self._sh = shared
        self.rank = rank
        self.size = shared.size

    @classmethod
    def create(cls, size: int, timeout: float = 20.0) -> List["FakeRing"]:
        sh = _FakeRingShared(size, timeout)
        return [cls(sh, r) for r in range(size)]

    def drop_next_message_to(self, rank: int) -> None:
        """Fault injection: the next message addressed to ``rank`` is lost."""
        with self._sh.lock:
            self._sh.drop_next_message_to.add(rank)

    def send_recv(self, tensors):
        if self.size == 1:
            return list(tensors)
        dst = (self.rank + 1) % self.size
        with self._sh.lock:
            dropped = dst in self._sh.drop_next_message_to
            if dropped:
                self._sh.drop_next_message_to.discard(dst)
        if not dropped:
            self._sh.queues[dst].put([t.detach().clone() for t in tensors])
        try:
            return self._sh.queues[self.rank].get(timeout=self._sh.timeout)
        except queue.Empty as e:
            raise RingTimeout(f"rank {self.rank}: nothing arrived from rank "
                              f"{(self.rank - 1) % self.size} within {self._sh.timeout}s") from e

    def barrier(self):
        try:
            self._sh.barrier.wait(timeout=self._sh.timeout)
        except threading.BrokenBarrierError as e:
            raise RingTimeout(f"rank {self.rank}: barrier broken (a peer never arrived)") from e


def run_fake_ring(size: int, fn: Callable[[RingComm], object], timeout: float = 20.0) -> list:
    """Run ``fn(comm)`` on ``size`` in-process ranks (threads); returns the per-rank results and
    re-raises the first exception of any rank."""
    comms = FakeRing.create(size, timeout)
    results: list = [None] * size
    errors: list = [None] * size

    def work(r):
        try:
            results[r] = fn(comms[r])
        except BaseException as e:  # noqa: BLE001 - reported to the caller below
            errors[r] = e
            comms[r]._sh.barrier.abort()

    threads = [threading.Thread(target=work, args=(r,), daemon=True) for r in range(size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for e in errors:
        if e is not None:
            raise e
    return results
