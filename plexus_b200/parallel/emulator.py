"""Host emulation of the peer-memory kernels, for testing the fused collectives without GPUs.

``parallel/symm.py`` (workspace layout, slot and flag addresses, regrowth) and
``parallel/fused.py`` (op numbering, buffer parity, one-shot and two-shot sequencing, row segments)
are host code that only ever runs against device kernels.  With the emulation enabled the same host
code runs on CPU ranks (gloo): a workspace is a POSIX shared-memory segment mapped by every rank of
the axis (the stand-in for a CUDA-IPC mapping), addresses are real addresses of those mappings, and
each kernel of ``csrc/kernels/comm_fused.cu`` - plus the push epilogues of the SpMM and the GEMM -
is restated in a few lines of torch on views of that memory, including the flag publication and
the bounded wait that ends in a status word.  Rows a kernel does not write (other owners' rows in
the reduce-scatter push) are filled with NaN so that any use of them shows up.

Enable with ``emulator.enable()`` (or ``PLEXUS_EMULATE_PEER_MEMORY=1``) before
``init(comm="fused", device="cpu")``.
"""

from __future__ import annotations

import ctypes
import os
import time
from multiprocessing import shared_memory
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

_enabled = os.environ.get("PLEXUS_EMULATE_PEER_MEMORY", "0") not in ("", "0")


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def active() -> bool:
    return _enabled


def _view(addr: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
    """Tensor over ``numel`` elements of ``dtype`` at a raw address of this process."""
    esz = torch.empty(0, dtype=dtype).element_size()
    raw = np.ctypeslib.as_array((ctypes.c_uint8 * (numel * esz)).from_address(addr))
    return torch.from_numpy(raw).view(dtype)


def _copy(dst_addr: int, src: torch.Tensor) -> None:
    src = src.contiguous()
    ctypes.memmove(dst_addr, src.data_ptr(), src.numel() * src.element_size())


class _Kernels:
    """The subset of the extension's API the peer-memory path uses."""

    def __init__(self):
        self._segments: Dict[int, shared_memory.SharedMemory] = {}

    # -- symmetric workspace ---------------------------------------------------------------
    def _map(self, shm: shared_memory.SharedMemory) -> int:
        addr = ctypes.addressof(ctypes.c_char.from_buffer(shm.buf))
        self._segments[addr] = shm
        return addr

    def symm_alloc(self, nbytes: int):
        shm = shared_memory.SharedMemory(create=True, size=int(nbytes))
        addr = self._map(shm)
        ctypes.memset(addr, 0, int(nbytes))
        return addr, shm.name.encode().ljust(64, b"\0")

    def symm_open(self, handle: bytes) -> int:
        return self._map(shared_memory.SharedMemory(name=bytes(handle).rstrip(b"\0").decode()))

    def symm_close(self, addr: int) -> None:
        self._segments.pop(addr).close()

    def symm_fill(self, addr: int, byte: int, nbytes: int) -> None:
        ctypes.memset(addr, int(byte), int(nbytes))

    def symm_view(self, addr: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        return _view(addr, numel, dtype)

    def symm_free(self, addr: int) -> None:
        shm = self._segments.pop(addr)
        shm.close()
        shm.unlink()

    # -- flags -----------------------------------------------------------------------------
    @staticmethod
    def _signal_and_wait(remote, local, epoch, timeout_ms, kernel_id, status) -> bool:
        for a in remote:
            ctypes.c_int32.from_address(a).value = int(epoch)
        deadline = time.time() + timeout_ms / 1e3
        for q, a in enumerate(local):
            flag = ctypes.c_int32.from_address(a)
            while flag.value < epoch:
                if time.time() > deadline:
                    if int(status[0]) == 0:
                        status[:5] = torch.tensor([1, kernel_id, q, epoch, flag.value], dtype=torch.int32)
                    return False
                time.sleep(0.0002)
        return True

    # -- kernels ---------------------------------------------------------------------------
    def push_copy(self, src: torch.Tensor, dst_ptrs: Sequence[int]) -> None:
        for a in dst_ptrs:
            _copy(a, src)

    @staticmethod
    def _ordered_sum(own, others, me, acc_dtype):
        """Sum in group-rank order (the local operand at position ``me``), like the kernels do, in
        ``acc_dtype``: every rank of the group then gets bitwise the same result."""
        terms = list(others)
        terms.insert(max(0, min(me, len(terms))) if me >= 0 else 0, own)
        acc = torch.zeros_like(own, dtype=acc_dtype)
        for t in terms:
            acc = acc + t.to(acc_dtype)
        return acc

    def reduce_slots(self, out, slot_ptrs, slot_ld, relu, mask, remote, local, epoch, timeout_ms, kid, status,
                     me=-1):
        if not self._signal_and_wait(remote, local, epoch, timeout_ms, kid, status):
            return
        rows, cols = out.shape
        acc_dtype = torch.float64 if out.dtype == torch.float64 else torch.float32
        others = [_view(a, rows * slot_ld, out.dtype).view(rows, slot_ld)[:, :cols] for a in slot_ptrs]
        self._finish(out, self._ordered_sum(out, others, me, acc_dtype), relu, mask)

    @staticmethod
    def _finish(out, acc, relu, mask):
        if relu:
            acc = torch.relu(acc)
        if mask is not None:
            acc = acc * (mask > 0)
        out.copy_(acc.to(out.dtype))

    def segment_reduce(self, mc_ptr, all_ptrs, me, seg, relu, mask, remote, local, epoch, timeout_ms, kid, status,
                       max_blocks=0):
        """Reduce this rank's segment of the symmetric buffer and write the result to every rank
        (what the switch does for the device kernel: sum of all ranks' partials, one set of bits)."""
        if not self._signal_and_wait(remote, local, epoch, timeout_ms, kid, status):
            return
        rows, cols = seg.shape
        off = seg.data_ptr() - all_ptrs[me]
        acc_dtype = torch.float64 if seg.dtype == torch.float64 else torch.float32
        parts = [_view(a + off, rows * cols, seg.dtype).view(rows, cols) for a in all_ptrs]
        acc = torch.zeros((rows, cols), dtype=acc_dtype)
        for t in parts:
            acc = acc + t.to(acc_dtype)
        if relu:
            acc = torch.relu(acc)
        if mask is not None:
            acc = acc * (mask > 0)
        res = acc.to(seg.dtype)
        for t in parts:
            t.copy_(res)

    def reduce_sentinel(self, out, slot_ptrs, slot_ld, relu, mask, timeout_ms, kid, status, me=-1, max_blocks=0):
        """Flag-free receive side: the slots hold 0xFF bytes where nothing has arrived; wait (bounded)
        until no element is the sentinel, sum in group-rank order, put the sentinel back."""
        rows, cols = out.shape
        esz = out.element_size()
        acc_dtype = torch.float64 if out.dtype == torch.float64 else torch.float32
        deadline = time.time() + timeout_ms / 1e3
        views = []
        for q, a in enumerate(slot_ptrs):
            raw = _view(a, rows * slot_ld * esz, torch.uint8).view(rows, slot_ld, esz)[:, :cols]
            while bool((raw == 0xFF).all(dim=2).any()):
                if time.time() > deadline:
                    if int(status[0]) == 0:
                        status[:5] = torch.tensor([1, kid, 40 + q, 0, 0], dtype=torch.int32)
                    return
                time.sleep(0.0002)
            views.append(_view(a, rows * slot_ld, out.dtype).view(rows, slot_ld)[:, :cols])
        self._finish(out, self._ordered_sum(out, views, me, acc_dtype), relu, mask)
        for a in slot_ptrs:
            _view(a, rows * slot_ld * esz, torch.uint8).view(rows, slot_ld * esz)[:, : cols * esz].fill_(0xFF)

    def reduce_slots_f32(self, out, slot_ptrs, op, remote, local, epoch, timeout_ms, kid, status, me=-1):
        if not self._signal_and_wait(remote, local, epoch, timeout_ms, kid, status):
            return
        n = out.numel()
        others = [_view(a, n, out.dtype) for a in slot_ptrs]
        if op == 0:
            out.copy_(self._ordered_sum(out, others, me, out.dtype))
        else:
            for other in others:
                out.copy_(torch.maximum(out, other))

    def gather_slots(self, src_ptrs, dst_ptrs, nbytes, remote, local, epoch, timeout_ms, kid, status):
        if not self._signal_and_wait(remote, local, epoch, timeout_ms, kid, status):
            return
        for s, d in zip(src_ptrs, dst_ptrs):
            ctypes.memmove(d, s, nbytes)

    def reduce_segment(self, out, row0, rows, slot_ptrs, slot_ld, relu, mask, bcast_ptrs, remote, local, epoch,
                       timeout_ms, kid, status, me=-1):
        if not self._signal_and_wait(remote, local, epoch, timeout_ms, kid, status):
            return
        cols = out.shape[1]
        seg = out[row0 : row0 + rows]
        acc_dtype = torch.float64 if out.dtype == torch.float64 else torch.float32
        others = [_view(a, rows * slot_ld, out.dtype).view(rows, slot_ld)[:, :cols] for a in slot_ptrs]
        acc = self._ordered_sum(seg, others, me, acc_dtype)
        self._finish(seg, acc, relu, None if mask is None else mask[row0 : row0 + rows])
        for a in bcast_ptrs:
            _view(a, rows * slot_ld, out.dtype).view(rows, slot_ld)[:, :cols].copy_(seg)

    def gather_segments(self, src_ptrs, dst_ptrs, nbytes, remote, local, epoch, timeout_ms, kid, status):
        if not self._signal_and_wait(remote, local, epoch, timeout_ms, kid, status):
            return
        for s, d, n in zip(src_ptrs, dst_ptrs, nbytes):
            ctypes.memmove(d, s, n)


class _Ops:
    """Stand-ins for ``ops/cuda.py``: the compute kernels with their push epilogues."""

    def __init__(self):
        self.launch_count = 0
        self._status: Optional[torch.Tensor] = None

    def _count(self, n: int) -> None:
        self.launch_count += n

    def status_buffer(self, device=None) -> torch.Tensor:
        if self._status is None:
            self._status = torch.zeros(8, dtype=torch.int32)
        return self._status

    def check_status(self, device=None) -> None:
        from .watchdog import raise_on_device_status

        raise_on_device_status(self.status_buffer())

    @staticmethod
    def _push(out: torch.Tensor, push_ptrs, push_ld, push_seg) -> None:
        seg, me = push_seg
        rows, cols = out.shape
        if not push_ptrs:
            return
        if seg == 0:  # one-shot: every row to every peer
            for a in push_ptrs:
                _view(a, rows * push_ld, out.dtype).view(rows, push_ld)[:, :cols].copy_(out)
            return
        # reduce-scatter: row r goes only to group rank r // seg; peers are listed without `me`
        for idx, a in enumerate(push_ptrs):
            owner = idx + (1 if idx >= me else 0)
            r0, r1 = min(owner * seg, rows), min((owner + 1) * seg, rows)
            if r1 > r0:
                _view(a, (r1 - r0) * push_ld, out.dtype).view(r1 - r0, push_ld)[:, :cols].copy_(out[r0:r1])
                out[r0:r1] = float("nan")  # the kernel never writes these rows locally

    def spmm_supports_tile_reduce(self, A, H, row_range=None) -> bool:
        return True

    def spmm(self, A, H, relu_mask=None, row_range=None, out_dtype=None, out=None, push_ptrs=(), push_ld=0,
             variant=None, push_seg=(0, 0), tile_reduce=None):
        from ..ops import reference

        fused = tile_reduce is not None and len(tile_reduce[0]) > 0
        res = reference.spmm(A, H, relu_mask=None if fused else relu_mask, row_range=row_range,
                             out_dtype=out_dtype).contiguous()
        if out is not None:
            out.copy_(res)
            res = out
        self._push(res, list(push_ptrs), push_ld, push_seg)
        if fused:
            self._sentinel_reduce(res, tile_reduce, push_ld, False, relu_mask)
        self._count(1)
        return res

    def _sentinel_reduce(self, res, tile_reduce, slot_ld, relu, mask):
        """The in-kernel all-reduce: the peers' partials sit in sentinel-kept slots (every byte 0xFF
        where nothing has arrived).  Wait (bounded) until no element of a slot is the sentinel, sum
        in group-rank order, apply ReLU / the mask, and put the sentinel back."""
        slots, me, timeout_ms = tile_reduce
        rows, cols = res.shape
        esz = res.element_size()
        acc_dtype = torch.float64 if res.dtype == torch.float64 else torch.float32
        deadline = time.time() + timeout_ms / 1e3
        views = []
        for q, a in enumerate(slots):
            raw = _view(a, rows * slot_ld * esz, torch.uint8).view(rows, slot_ld, esz)[:, :cols]
            while bool((raw == 0xFF).all(dim=2).any()):
                if time.time() > deadline:
                    st = self.status_buffer()
                    if int(st[0]) == 0:
                        st[:5] = torch.tensor([1, 6, 30 + q, 0, 0], dtype=torch.int32)
                    return
                time.sleep(0.0002)
            views.append(_view(a, rows * slot_ld, res.dtype).view(rows, slot_ld)[:, :cols])
        _Kernels._finish(res, _Kernels._ordered_sum(res, views, me, acc_dtype), relu, mask)
        for a in slots:
            _view(a, rows * slot_ld * esz, torch.uint8).view(rows, slot_ld * esz)[:, : cols * esz].fill_(0xFF)

    def gemm(self, a, b, trans_a=False, trans_b=False, relu=False, out_dtype=None, variant=0, push_ptrs=(),
             push_ld=0, relu_mask=None, push_seg=(0, 0), out=None, tile_reduce=None):
        from ..ops import reference

        fused = tile_reduce is not None and len(tile_reduce[0]) > 0
        # with the in-kernel all-reduce the activation and the mask come after the sum
        res = reference.gemm(a, b, trans_a=trans_a, trans_b=trans_b, relu=relu and not fused,
                             out_dtype=out_dtype).contiguous()
        if relu_mask is not None and not fused:
            res = reference.relu_backward(res, relu_mask)
        if out is not None:
            out.copy_(res)
            res = out
        self._push(res, list(push_ptrs), push_ld, push_seg)
        if fused:
            self._sentinel_reduce(res, tile_reduce, push_ld, relu, relu_mask)
        self._count(1)
        return res

    def relu_backward(self, grad, out):
        from ..ops import reference

        return reference.relu_backward(grad, out)

    # -- cross-entropy with the exchange inside the kernels -------------------------------------
    def xent_stats(self, logits, class_offset, num_classes, target=None, row_offset=0, num_nodes=0, weight=None,
                   push_ptrs=()):
        from ..ops import reference

        stats, loss = reference.xent_stats(logits, class_offset, num_classes, target, row_offset, num_nodes, weight)
        stats = stats.contiguous()
        for a in push_ptrs:  # the kernel stores every pair into this rank's slot on each peer as well
            _copy(a, stats)
        self._count(1)
        return stats, loss

    def xent_combine_ptrs(self, logits, target, pair_ptrs, row_offset, class_offset, num_nodes, weight=None,
                          sync=None, like=None):
        """``like``: a statistics tensor of this rank (gives dtype and row count of the pairs)."""
        from ..ops import reference

        if sync is not None:
            remote, local, epoch, timeout_ms = sync
            if not C._signal_and_wait(remote, local, epoch, timeout_ms, 5, self.status_buffer()):
                R = logits.shape[0]
                return torch.zeros((2, R), dtype=like.dtype), torch.zeros((), dtype=like.dtype)
        R = logits.shape[0]
        pairs = torch.stack([_view(a, 2 * R, like.dtype).view(2, R).clone() for a in pair_ptrs])
        self._count(1)
        return reference.xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, weight)


C = _Kernels()
ops = _Ops()
