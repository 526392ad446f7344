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

    def symm_clear(self, addr: int, nbytes: int) -> None:
        ctypes.memset(addr, 0, int(nbytes))

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
            self._tile_reduce_rows(res, tile_reduce, push_ld, relu_mask)
        self._count(1)
        return res

    def _tile_reduce_rows(self, res, tile_reduce, slot_ld, mask):
        """The SpMM's in-kernel all-reduce: per exchange tile, add the rows pushed to the peers'
        counters, wait (bounded) for the peers' counts, sum in group-rank order, clear the counters."""
        slots, remote_sig, local_sig, me, timeout_ms, tile_rows, _local_done = tile_reduce
        rows, cols = res.shape
        acc_dtype = torch.float64 if res.dtype == torch.float64 else torch.float32
        tiles = [(t0, min(tile_rows, rows - t0)) for t0 in range(0, rows, tile_rows)]
        for T, (t0, n) in enumerate(tiles):
            for a in remote_sig:
                c = ctypes.c_int32.from_address(a + 4 * T)
                c.value = c.value + n  # the only writer of this counter during the op
        deadline = time.time() + timeout_ms / 1e3
        for T, (t0, n) in enumerate(tiles):
            for q, a in enumerate(local_sig):
                c = ctypes.c_int32.from_address(a + 4 * T)
                while c.value < n:
                    if time.time() > deadline:
                        st = self.status_buffer()
                        if int(st[0]) == 0:
                            st[:5] = torch.tensor([1, 7, 20 + q, n, c.value], dtype=torch.int32)
                        return
                    time.sleep(0.0002)
            seg = res[t0 : t0 + n]
            others = [_view(a, rows * slot_ld, res.dtype).view(rows, slot_ld)[t0 : t0 + n, :cols] for a in slots]
            _Kernels._finish(seg, _Kernels._ordered_sum(seg, others, me, acc_dtype), False,
                             None if mask is None else mask[t0 : t0 + n])
            for a in local_sig:
                ctypes.c_int32.from_address(a + 4 * T).value = 0

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
            self._tile_reduce(res, tile_reduce, push_ld, relu, relu_mask, signal_index=0)
        self._count(1)
        return res

    def _tile_reduce(self, res, tile_reduce, slot_ld, relu, mask, signal_index):
        """The in-kernel all-reduce with the whole matrix as one tile: publish one signal per peer
        (value ``base + 1``), wait for the peers' signals (bounded), sum in group-rank order."""
        slots, remote_sig, local_sig, base, me, timeout_ms = tile_reduce[:6]
        for a in remote_sig:
            ctypes.c_int32.from_address(a + 4 * signal_index).value = int(base) + 1
        deadline = time.time() + timeout_ms / 1e3
        for q, a in enumerate(local_sig):
            flag = ctypes.c_int32.from_address(a + 4 * signal_index)
            while flag.value - (int(base) + 1) < 0:
                if time.time() > deadline:
                    st = self.status_buffer()
                    if int(st[0]) == 0:
                        st[:5] = torch.tensor([1, 6, 20 + q, int(base) + 1, flag.value], dtype=torch.int32)
                    return
                time.sleep(0.0002)
        rows, cols = res.shape
        acc_dtype = torch.float64 if res.dtype == torch.float64 else torch.float32
        others = [_view(a, rows * slot_ld, res.dtype).view(rows, slot_ld)[:, :cols] for a in slots]
        _Kernels._finish(res, _Kernels._ordered_sum(res, others, me, acc_dtype), relu, mask)

    def relu_backward(self, grad, out):
        from ..ops import reference

        return reference.relu_backward(grad, out)


C = _Kernels()
ops = _Ops()
