"""Host-side model of the symmetric-memory protocol used by the fused ring (a race detector that
needs no GPU).

The kernels of one rank run in stream order; different ranks run concurrently and only meet at the
flag barrier. A schedule is safe if no rank ever writes a buffer while another rank may still be
reading or writing it. :func:`check_schedule` explores *every* interleaving of N ranks that the
barriers allow (each kernel is a begin and an end event with read and write sets) and reports the
first conflict. The programs below mirror ``parallel/symm.py``, ``ops/decode.py`` and the sharded
weights of ``models/params.py``; the tests run
them for small N and several consecutive calls, and also check that removing a barrier or the
double buffering is detected.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import FrozenSet, List, Optional, Tuple


@dataclass(frozen=True)
class Op:
    kind: str                       # "kernel" or "barrier"
    reads: FrozenSet[Tuple] = frozenset()
    writes: FrozenSet[Tuple] = frozenset()
    name: str = ""


def kernel(name, reads=(), writes=()) -> Op:
    return Op("kernel", frozenset(reads), frozenset(writes), name)


BARRIER = Op("barrier", name="barrier")


def ring_forward_program(rank: int, n: int, calls: int, double_buffer: bool = True, barrier: bool = True) -> List[Op]:
    """Forward of ``SymmRing``: stage own KV into slot (call & 1), barrier, then N steps; the kernel
    of step i reads slab (i-1)&1 and pulls block (rank-i-1) from its owner into slab i&1."""
    ops: List[Op] = []
    for c in range(calls):
        slot = (c & 1) if double_buffer else 0
        ops.append(kernel(f"stage{c}", writes=[("own", rank, slot)]))
        if barrier:
            ops.append(BARRIER)
        for i in range(n):
            reads, writes = [], []
            if i > 0:
                reads.append(("slab", rank, (i - 1) & 1))
            if i + 1 < n:
                src = (rank - i - 1) % n
                reads.append(("own", src, slot))
                writes.append(("slab", rank, i & 1))
            ops.append(kernel(f"step{c}.{i}", reads, writes))
    return ops


def ring_backward_program(rank: int, n: int, calls: int, second_barrier: bool = True) -> List[Op]:
    """Backward: zero own accumulator, stage KV, barrier, steps that reduce into the owner's
    accumulator, barrier, cast own accumulator."""
    ops: List[Op] = []
    for c in range(calls):
        slot = c & 1
        ops.append(kernel(f"zero{c}", writes=[("acc", rank)]))
        ops.append(kernel(f"stage{c}", writes=[("own", rank, slot)]))
        ops.append(BARRIER)
        for i in range(n):
            blk = (rank - i) % n
            reads, writes = [], [("acc+", blk)]  # reductions commute: tracked as a separate class
            if i > 0:
                reads.append(("slab", rank, (i - 1) & 1))
            if i + 1 < n:
                reads.append(("own", (rank - i - 1) % n, slot))
                writes.append(("slab", rank, i & 1))
            ops.append(kernel(f"bstep{c}.{i}", reads, writes))
        if second_barrier:
            ops.append(BARRIER)
        ops.append(kernel(f"cast{c}", reads=[("acc", rank)]))
    return ops


def decode_program(rank: int, n: int, calls: int, double_buffer: bool = True) -> List[Op]:
    """Decode merge: store the partial into slot `rank` of every inbox, barrier, merge own inbox."""
    ops: List[Op] = []
    for c in range(calls):
        slot = (c & 1) if double_buffer else 0
        ops.append(kernel(f"push{c}", writes=[("inbox", r, slot, rank) for r in range(n)]))
        ops.append(BARRIER)
        ops.append(kernel(f"merge{c}", reads=[("inbox", rank, slot, s) for s in range(n)]))
    return ops


def fsdp_program(rank: int, n: int, steps: int, gemms: int = 3, sync_after_update: bool = True,
                 reduce_before_update: bool = True) -> List[Op]:
    """Training steps with row-sharded weights (``models/params.py``): the GEMMs of a step read every
    peer's bf16 shard in place (copy CTAs) and write the local landing area; the gradient reduction
    is a collective every rank enters after its own backward; the optimizer then rewrites the own
    shard; a small collective after the update keeps peers from starting the next step early."""
    ops: List[Op] = []
    for t in range(steps):
        for g in range(gemms):
            ops.append(kernel(f"gemm{t}.{g}", reads=[("shard", s) for s in range(n)] + [("landing", rank)],
                              writes=[("landing", rank)]))
        if reduce_before_update:
            ops.append(BARRIER)   # gradient reduce-scatter / all-reduce
        ops.append(kernel(f"adamw{t}", writes=[("shard", rank)]))
        if sync_after_update:
            ops.append(BARRIER)   # sync token
    return ops


def _conflict(a_reads, a_writes, b_reads, b_writes) -> Optional[Tuple]:
    def base(x):  # ("acc+", r) and ("acc", r) name the same memory
        return ("acc",) + x[1:] if x[0] == "acc+" else x

    for w in a_writes:
        for other in list(b_reads) + list(b_writes):
            if base(w) == base(other):
                if w[0] == "acc+" and other[0] == "acc+":
                    continue  # concurrent reductions into the same accumulator are fine
                return w
    for r in a_reads:
        for w in b_writes:
            if base(r) == base(w):
                return r
    return None


def check_schedule(programs: List[List[Op]]) -> Optional[str]:
    """Explore all interleavings; return a description of the first race found, or ``None``."""
    n = len(programs)
    # state: per rank (pc, running) where running means the kernel at pc has begun but not ended
    start = tuple((0, False) for _ in range(n))
    seen = {start}
    stack = [start]
    while stack:
        st = stack.pop()
        for r in range(n):
            pc, running = st[r]
            if pc >= len(programs[r]):
                continue
            op = programs[r][pc]
            if op.kind == "barrier":
                # passes only when every rank has reached its matching barrier (same ordinal)
                k = sum(1 for o in programs[r][:pc] if o.kind == "barrier")
                ok = True
                for s in range(n):
                    spc, srun = st[s]
                    arrived = sum(1 for o in programs[s][:spc] if o.kind == "barrier")
                    at_barrier = spc < len(programs[s]) and programs[s][spc].kind == "barrier" and not srun
                    if not (arrived > k or (arrived == k and at_barrier)):
                        ok = False
                        break
                if not ok:
                    continue
                nxt = list(st)
                nxt[r] = (pc + 1, False)
            elif not running:
                # begin: conflicts with kernels running on other ranks?
                for s in range(n):
                    if s == r:
                        continue
                    spc, srun = st[s]
                    if srun:
                        o2 = programs[s][spc]
                        c = _conflict(op.reads, op.writes, o2.reads, o2.writes)
                        if c is not None:
                            return f"rank {r} {op.name} races with rank {s} {o2.name} on {c}"
                nxt = list(st)
                nxt[r] = (pc, True)
            else:
                nxt = list(st)
                nxt[r] = (pc + 1, False)
            t = tuple(nxt)
            if t not in seen:
                seen.add(t)
                stack.append(t)
    return None


def check_row_exchange(n: int, rows: int, launches: int, slots: int = 2) -> Optional[str]:
    """The one-launch decode exchange (``decode_merge_exchange_kernel``): in launch ``e`` CTA ``row`` of every rank
    stores its partial into slot ``e % slots`` of every rank's inbox and raises the row's flag there, waits for the
    row's flag of launch ``e`` from every rank and merges the row of its own inbox; a rank starts launch ``e + 1``
    when all its rows are done. There is no barrier: ranks only meet row by row. Explores every interleaving of
    these steps and returns a description of the first store that lands in an inbox slot whose previous content has
    not been merged yet, or ``None``."""
    # per rank: (launch, phases) with phase 0 = nothing yet, 1 = stored and flagged (waiting), 2 = merged
    start = tuple((0, (0,) * rows) for _ in range(n))
    seen, stack = {start}, [start]
    while stack:
        st = stack.pop()
        for r in range(n):
            e, ph = st[r]
            if e >= launches:
                continue
            for row in range(rows):
                if ph[row] == 0:  # store + flag
                    for t in range(n):
                        te, tph = st[t]
                        merged = te + (1 if te < launches and tph[row] == 2 else 0)  # launches whose row t has merged
                        if merged < e - slots + 1:
                            return (f"rank {r} launch {e} row {row} overwrites slot {e % slots} of rank {t}, "
                                    f"which has merged only {merged} launches")
                    nph = ph[:row] + (1,) + ph[row + 1:]
                elif ph[row] == 1:  # wait for the row of every rank, then merge
                    if not all(se > e or (se == e and sph[row] >= 1) for se, sph in st):
                        continue
                    nph = ph[:row] + (2,) + ph[row + 1:]
                else:
                    continue
                nst = list(st)
                nst[r] = (e + 1, (0,) * rows) if all(x == 2 for x in nph) else (e, nph)
                t = tuple(nst)
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
    return None
