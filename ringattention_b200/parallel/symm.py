"""Symmetric memory over NVLink and the fused ring schedule built on it.

The reference leaves communication to XLA (``lax.ppermute`` -> NCCL collective-permute,
ringattention_jax.py:47,85-86). Here every rank of the ring owns device buffers that all other
ranks of the node map into their address space (CUDA IPC), so kernels address peer memory
directly:

* forward: the attention kernel of ring step t carries copy CTAs that pull the KV block of step
  t+1 from its *owner* (NVSwitch gives every pair full bandwidth, so nothing is forwarded hop by
  hop) into one of two local slabs while the other CTAs compute on the block of step t;
* backward: K/V are pulled the same way, and the dK/dV contribution of this rank for block j is
  added straight into rank j's fp32 accumulator by system-scope vector reductions in the kernel
  epilogue;
* synchronisation: a flag barrier with bounded waits (``ra_symm_barrier``) before the first pull
  and after the last reduction. A rank that never arrives makes the others record a timeout in the
  status word instead of hanging; the next ``check_status`` raises.

Only plain loads, stores and reductions touch peer memory; nothing is broadcast through the switch.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib, flash
from ..ops import kernels as K
from ..utils.tracing import phase

c_vp = ctypes.c_void_p


class _RawCudaBuffer:
    """Adapter that lets ``torch.as_tensor`` wrap a raw device pointer without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_ptr(ptr: int, nbytes: int, device) -> torch.Tensor:
    """uint8 tensor aliasing ``nbytes`` of device memory at ``ptr`` (local or peer-mapped)."""
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=device)


class SymmBuffer:
    """One symmetric allocation: ``local`` is this rank's memory, ``peer_ptrs[r]`` the address of
    rank r's copy in this process (``peer_ptrs[rank]`` is the local pointer)."""

    def __init__(self, nbytes: int, group, device):
        self.nbytes = nbytes
        self.device = device
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        lib = _lib.lib()
        p = c_vp()
        _lib.call("ra_symm_alloc", ctypes.c_ulonglong(nbytes), ctypes.byref(p), n_kernels=0)
        self.ptr = int(p.value)
        handle = ctypes.create_string_buffer(64)
        _lib.call("ra_ipc_get_handle", c_vp(self.ptr), handle, n_kernels=0)
        handles: List[Optional[bytes]] = [None] * self.size
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.peer_ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self.ptr)
                continue
            q = c_vp()
            _lib.call("ra_ipc_open", ctypes.create_string_buffer(h, 64), ctypes.byref(q), n_kernels=0)
            self.peer_ptrs.append(int(q.value))
            self._opened.append(int(q.value))
        self.local = tensor_from_ptr(self.ptr, nbytes, device)
        self._lib = lib

    def peer_tensor(self, r: int) -> torch.Tensor:
        return tensor_from_ptr(self.peer_ptrs[r], self.nbytes, self.device)

    def close(self) -> None:
        for q in self._opened:
            self._lib.ra_ipc_close(c_vp(q))
        self._opened = []
        if self.ptr:
            self._lib.ra_symm_free(c_vp(self.ptr))
            self.ptr = 0


class SymmRing:
    """Symmetric buffers, barrier and the fused forward/backward ring schedule of one ``sp`` group."""

    def __init__(self, group, device, timeout_s: Optional[float] = None, copy_ctas: int = 16):
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.timeout_ns = int(float(os.environ.get("RINGATTN_B200_BARRIER_TIMEOUT_S",
                                                   timeout_s if timeout_s is not None else 10.0)) * 1e9)
        self.copy_ctas = copy_ctas
        self.overlap = True  # False: pull each block with a separate copy kernel before its step (for measurements)
        self.calls = 0
        self._bufs: Dict[str, SymmBuffer] = {}
        self._local: Dict[str, torch.Tensor] = {}
        self.flags = SymmBuffer(256, group, self.device)
        self._flag_ptrs = torch.tensor(self.flags.peer_ptrs, dtype=torch.int64, device=self.device)
        # barrier count kept on the device, so that a barrier recorded in a CUDA graph stays valid on replay
        self._epoch_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._ptr_cache: Dict[str, tuple] = {}
        dist.barrier(group=group)

    # ------------------------------------------------------------------ plumbing
    def buffer(self, name: str, nbytes: int) -> SymmBuffer:
        """Symmetric buffer ``name`` of at least ``nbytes`` (collective: all ranks call it with the
        same sizes in the same order; it is re-created when it has to grow)."""
        b = self._bufs.get(name)
        if b is None or b.nbytes < nbytes:
            if b is not None:
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.group)
                b.close()
            b = SymmBuffer((nbytes + 255) // 256 * 256, self.group, self.device)
            self._bufs[name] = b
        return b

    def scratch(self, name: str, nbytes: int) -> torch.Tensor:
        t = self._local.get(name)
        if t is None or t.numel() < nbytes:
            t = torch.empty((nbytes + 255) // 256 * 256, dtype=torch.uint8, device=self.device)
            self._local[name] = t
        return t

    def scratch_zeros(self, name: str, nbytes: int) -> torch.Tensor:
        """Local device words that start at zero and keep their contents between calls (launch counters)."""
        t = self._local.get(name)
        if t is None:
            t = torch.zeros((nbytes + 255) // 256 * 256, dtype=torch.uint8, device=self.device)
            self._local[name] = t
        return t

    def barrier(self) -> None:
        """Stream-ordered flag barrier across the ring; a missing peer ends in a status code."""
        _lib.call("ra_symm_barrier", c_vp(self._flag_ptrs.data_ptr()), self.rank, self.size,
                  ctypes.c_uint(0), ctypes.c_ulonglong(self.timeout_ns),
                  c_vp(_lib.status_tensor(self.device).data_ptr()), _lib.stream_ptr(),
                  c_vp(self._epoch_dev.data_ptr()))

    def peer_ptr_table(self, name: str) -> torch.Tensor:
        """Device array with every rank's address of symmetric buffer ``name`` (cached)."""
        b = self._bufs[name]
        hit = self._ptr_cache.get(name)
        if hit is None or hit[0] != b.ptr:  # (re)allocated since the table was built
            hit = (b.ptr, torch.tensor(b.peer_ptrs, dtype=torch.int64, device=self.device))
            self._ptr_cache[name] = hit
        return hit[1]

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        for b in self._bufs.values():
            b.close()
        self._bufs = {}
        self.flags.close()

    # ------------------------------------------------------------------ KV staging
    def _stage_kv(self, k, v):
        """Copy this rank's K/V into its symmetric slot ``(B, S, 2, H, D)`` for this call."""
        B, S, H, D = k.shape
        nb = B * S * 2 * H * D * 2
        own = self.buffer("kv_own", 2 * nb)
        slot = self.calls & 1
        self.calls += 1
        view = own.local[slot * nb:(slot + 1) * nb].view(torch.bfloat16).view(B, S, 2, H, D)
        with phase("ring_stage_kv"):
            self._copy_rows(k, view[:, :, 0])
            self._copy_rows(v, view[:, :, 1])
        slabs = self.scratch("kv_slabs", 2 * nb)
        return own, slot, nb, slabs

    @staticmethod
    def _copy_rows(src: torch.Tensor, dst: torch.Tensor) -> None:
        """``dst[b, s] = src[b, s]`` for ``(B, S, H, D)`` views whose ``(H, D)`` block is contiguous and whose
        tokens are evenly spaced (a slice of a fused QKV projection): one row copy at memory speed."""
        B, S, H, D = src.shape
        ok = lambda t: (t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == S * t.stride(1)
                        and (t.stride(1) * 2) % 16 == 0 and t.data_ptr() % 16 == 0)
        if (H * D * 2) % 16 or not (ok(src) and ok(dst)):
            dst.copy_(src)
            return
        _lib.call("ra_copy_rows", c_vp(src.data_ptr()), c_vp(dst.data_ptr()), ctypes.c_longlong(B * S),
                  ctypes.c_longlong(H * D * 2), ctypes.c_longlong(src.stride(1) * 2),
                  ctypes.c_longlong(dst.stride(1) * 2), _lib.stream_ptr())

    def _slab_views(self, slabs, i, nb, B, S, H, D):
        t = slabs[i * nb:(i + 1) * nb].view(torch.bfloat16).view(B, S, 2, H, D)
        return t[:, :, 0], t[:, :, 1]

    def _maybe_serial_copy(self, cp: dict) -> dict:
        """With ``overlap`` off, do the pull with a stand-alone copy kernel now (stream order puts it
        before the step that would have carried it) and hand the attention kernel no copy job."""
        if self.overlap:
            return cp
        _lib.call("ra_peer_copy", c_vp(cp["copy_src"]), c_vp(cp["copy_dst"]), ctypes.c_longlong(cp["copy_bytes"]),
                  64, _lib.stream_ptr())
        return {}

    # ------------------------------------------------------------------ fused forward
    def forward(self, q, k, v, plan, out=None):
        B, Sq, H, D = q.shape
        S = k.shape[1]
        own, slot, nb, slabs = self._stage_kv(k, v)
        with phase("ring_start_barrier"):
            self.barrier()
        steps = plan.active
        n = len(steps)
        if out is None:
            out = torch.empty(B, Sq, H, D, device=q.device, dtype=torch.bfloat16)
        lse = torch.empty(B, H, Sq, device=q.device, dtype=torch.float32)
        o_acc = None
        if n > 1:
            o_acc = self.scratch("o_acc", B * Sq * H * D * 4).view(torch.float32)[:B * Sq * H * D].view(B, Sq, H, D)
        if n == 0:
            out.zero_()
            lse.fill_(float("-inf"))
            return out, lse
        have_prev = False
        for i, st in enumerate(steps):
            if st.block == self.rank:
                kk, vv = k, v
            else:
                kk, vv = self._slab_views(slabs, (i - 1) & 1, nb, B, S, H, D)
            cp = {}
            if i + 1 < n and steps[i + 1].block != self.rank:
                cp = dict(copy_src=own.peer_ptrs[steps[i + 1].block] + slot * nb,
                          copy_dst=slabs.data_ptr() + (i & 1) * nb, copy_bytes=nb, copy_ctas=self.copy_ctas)
                cp = self._maybe_serial_copy(cp)
            last = i == n - 1
            flash.flash_fwd(q, kk, vv, st.mask, o_prev=o_acc if have_prev else None,
                            lse_prev=lse if have_prev else None, out=out if last else o_acc,
                            lse_out=lse, **cp)
            have_prev = True
        return out, lse

    # ------------------------------------------------------------------ fused backward
    def backward(self, q, k, v, dout, lse2, delta, plan, dq_acc, dk, dv):
        B, Sq, H, D = q.shape
        S = k.shape[1]
        nacc = B * S * 2 * H * D * 4
        acc = self.buffer("dkv_acc", nacc)
        with phase("ring_zero_dkv_acc"):
            acc.local[:nacc].zero_()
        own, slot, nb, slabs = self._stage_kv(k, v)
        with phase("ring_start_barrier"):
            self.barrier()
        steps = plan.active
        n = len(steps)
        for i, st in enumerate(steps):
            if st.block == self.rank:
                kk, vv = k, v
            else:
                kk, vv = self._slab_views(slabs, (i - 1) & 1, nb, B, S, H, D)
            tgt = acc.local if st.block == self.rank else acc.peer_tensor(st.block)
            t5 = tgt[:nacc].view(torch.float32).view(B, S, 2, H, D)
            cp = {}
            if i + 1 < n and steps[i + 1].block != self.rank:
                cp = dict(copy_src=own.peer_ptrs[steps[i + 1].block] + slot * nb,
                          copy_dst=slabs.data_ptr() + (i & 1) * nb, copy_bytes=nb, copy_ctas=self.copy_ctas)
                cp = self._maybe_serial_copy(cp)
            flash.flash_bwd(q, kk, vv, dout, lse2, delta, st.mask, dq_acc, t5[:, :, 0], t5[:, :, 1],
                            flash.DKV_REDUCE_FP32, **cp)
        with phase("ring_end_barrier"):
            self.barrier()
        a5 = acc.local[:nacc].view(torch.float32).view(B * S, 2, H * D)
        with phase("ring_cast_dkv"):
            for which, dst in ((0, dk), (1, dv)):
                sd = dst.stride()
                if sd[3] == 1 and sd[2] == D and sd[0] == S * sd[1]:
                    d2 = dst.as_strided((B * S, H * D), (sd[1], 1), dst.storage_offset())
                    K.cast_f32_to_bf16(a5[:, which], d2)
                else:
                    dst.copy_(a5[:, which].view(B, S, H, D))


def peer_bandwidth_probe(ring: SymmRing, nbytes: int = 1 << 30, ctas: int = 64, iters: int = 5) -> dict:
    """Measure peer-copy bandwidth (pull from the next rank) and barrier latency with CUDA events."""
    buf = ring.buffer("probe", nbytes)
    dst = ring.scratch("probe_dst", nbytes)
    peer = (ring.rank + 1) % ring.size
    ring.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(2):
        _lib.call("ra_peer_copy", c_vp(buf.peer_ptrs[peer]), c_vp(dst.data_ptr()),
                  ctypes.c_longlong(nbytes), ctas, _lib.stream_ptr())
    e0.record()
    for _ in range(iters):
        _lib.call("ra_peer_copy", c_vp(buf.peer_ptrs[peer]), c_vp(dst.data_ptr()),
                  ctypes.c_longlong(nbytes), ctas, _lib.stream_ptr())
    e1.record()
    torch.cuda.synchronize()
    copy_ms = e0.elapsed_time(e1) / iters
    e0.record()
    for _ in range(20):
        ring.barrier()
    e1.record()
    torch.cuda.synchronize()
    return {"pull_gbs": nbytes / copy_ms / 1e6, "ctas": ctas, "barrier_us": e0.elapsed_time(e1) / 20 * 1e3}
