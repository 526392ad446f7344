"""Symmetric peer-memory workspaces, one per grid axis this rank belongs to.

A workspace is one ``cudaMalloc`` per rank whose CUDA-IPC handle is exchanged over the axis'
process group, so every rank holds a device pointer into every peer's buffer and kernels can
store into / load from peer memory directly over NVLink.  Layout of each rank's buffer::

    [ flags: int32[2][8] (1 KiB) | buffer 0: p slots | buffer 1: p slots | sentinel buffer 0 | sentinel buffer 1 ]

Slot ``s`` of a buffer receives data from group rank ``s``.  The op counter ("epoch") of an axis
selects buffer ``epoch % 2``; see ``csrc/kernels/comm_fused.cu`` for the flag protocol and why
double buffering is enough.  The *sentinel* buffers serve the all-reduces that the compute kernels
finish themselves: they hold 0xFF bytes wherever nothing has arrived, the receiving kernel
recognises arrived bf16 data by itself and puts the sentinel back after use, so these ops need
neither flags nor fences (``csrc/include/sentinel_reduce.cuh``).  Workspaces grow on demand (a
collective operation: every rank of the axis asks for the same size at the same point of the
program).

Beside the slot workspace an axis can own a *symmetric buffer* (``ensure_symmetric``): one
allocation at the same offset on every rank, bound to an NVLink multicast address where the fabric
allows it, which the segment-reduce form of the all-reduce works on (``csrc/kernels/nvls_reduce.cu``).
"""

from __future__ import annotations

import hashlib
import os
import socket
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from . import backend


def _C():
    """The kernels bound by ``runtime.init`` (the extension, or its host emulation in tests)."""
    return backend.C()


def _device_sync() -> None:
    if not backend.emulated:
        torch.cuda.synchronize()

MAX_GROUP = 8
FLAG_BYTES = 1024
DEFAULT_TIMEOUT_MS = 5000.0
# Bind the symmetric buffers to an NVLink multicast object (in-switch reduction).  Switch it off for
# runs in which a rank may exit while others still use the buffers (fault-injection tests).
NVLS = os.environ.get("PLEXUS_NVLS", "1") != "0"


# PLEXUS_DEBUG=1: the push epilogues of the SpMM / GEMM kernels check every store into a peer's
# receive slot against the slot size on the device (reported through the status words).
DEBUG = os.environ.get("PLEXUS_DEBUG", "0") not in ("", "0")


class PushList(list):
    """Push target addresses plus, in a debug run, the capacity of each target slot in bytes."""

    limit_bytes = 0


class AxisComm:
    def __init__(self, group):
        self.group = group
        self.p = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.p > MAX_GROUP:
            raise ValueError(f"peer-memory collectives support at most {MAX_GROUP} ranks per axis")
        self.peers = [q for q in range(self.p) if q != self.rank]
        # CUDA-IPC handles only open inside one host: an axis that spans hosts keeps the library path.
        # Host names are compared through a fixed-size byte all-gather (the same collective the
        # workspace set-up uses for the IPC handles).
        host = os.environ.get("PLEXUS_HOST_ID") or socket.gethostname()
        dev = (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl"
               else torch.device("cpu"))
        mine = torch.frombuffer(bytearray(hashlib.sha1(host.encode()).digest()[:16]), dtype=torch.uint8).to(dev)
        allh = torch.empty(self.p * 16, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allh, mine, group=group)
        allh = allh.cpu().view(self.p, 16)
        self.same_host = bool((allh == allh[0]).all())
        self.epoch = 0
        self.slot_bytes = 0
        self.sslot_bytes = 0  # slot size of the sentinel buffers
        self.local_ptr = 0
        self.ptrs: List[int] = []
        self.timeout_ms = DEFAULT_TIMEOUT_MS
        # symmetric buffer of the segment-reduce form (see ensure_symmetric)
        self.sym_bytes = 0
        self.sym_ptrs: List[int] = []  # every rank's buffer, group-rank order
        self.sym_mc = 0                # multicast address (0: none, plain peer loads / stores)
        self._sym_tensor = None        # torch symmetric-memory tensor that owns the buffer, or
        self._sym_local = 0            # the local CUDA-IPC allocation

    # -- allocation ---------------------------------------------------------------------
    def ensure(self, slot_bytes: int = 0, sentinel_bytes: int = 0) -> None:
        """Make the flagged slots at least ``slot_bytes`` and the sentinel slots at least
        ``sentinel_bytes`` large (collective over the axis when something has to grow)."""
        if not self.same_host:
            raise RuntimeError("peer-memory workspace requested for an axis that spans hosts")
        slot_bytes = max(self.slot_bytes, (int(slot_bytes) + 1023) // 1024 * 1024)
        sentinel_bytes = max(self.sslot_bytes, (int(sentinel_bytes) + 1023) // 1024 * 1024)
        if slot_bytes == self.slot_bytes and sentinel_bytes == self.sslot_bytes and self.ptrs:
            return
        C = _C()
        dev = (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl"
               else torch.device("cpu"))
        # nobody may still be using the old workspace
        _device_sync()
        dist.barrier(group=self.group)
        self.release()
        plain = 2 * self.p * slot_bytes
        total = FLAG_BYTES + plain + 2 * self.p * sentinel_bytes
        ptr, handle = C.symm_alloc(total)
        if sentinel_bytes:
            C.symm_fill(ptr + FLAG_BYTES + plain, 0xFF, 2 * self.p * sentinel_bytes)
        mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8).to(dev)
        allh = torch.empty(self.p * 64, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allh, mine, group=self.group)
        allh = allh.cpu().view(self.p, 64)
        self.ptrs = []
        for q in range(self.p):
            self.ptrs.append(ptr if q == self.rank else C.symm_open(bytes(allh[q].tolist())))
        self.local_ptr, self.slot_bytes, self.sslot_bytes = ptr, slot_bytes, sentinel_bytes
        _device_sync()
        dist.barrier(group=self.group)

    def release(self) -> None:
        """Unmap the peers' buffers, then (after everybody did) free the local one."""
        if not self.ptrs:
            return
        C = _C()
        for q, ptr in enumerate(self.ptrs):
            if q != self.rank:
                C.symm_close(ptr)
        try:
            dist.barrier(group=self.group)  # no importer may still map a buffer that gets freed
        except Exception:
            pass
        C.symm_free(self.local_ptr)
        self.ptrs, self.local_ptr = [], 0
        self.slot_bytes = self.sslot_bytes = 0

    # -- symmetric buffer (segment-reduce form) ---------------------------------------------
    def ensure_symmetric(self, nbytes: int) -> None:
        """One buffer of at least ``nbytes`` at the same offset on every rank of the axis, for the
        all-reduce that reduces inside the NVSwitch (``csrc/kernels/nvls_reduce.cu``).

        With ``PLEXUS_NVLS`` on (default) the memory comes from torch's symmetric-memory allocator,
        which maps every peer's buffer and, where the fabric allows it, binds them to one multicast
        address; the allocator is all that is used of it, the kernels are this package's.  If that
        fails or with ``PLEXUS_NVLS=0`` the buffer is a CUDA-IPC allocation like the slot workspace
        and the kernel reduces with plain peer loads and stores.  Collective when it has to grow.
        """
        if not self.same_host:
            raise RuntimeError("peer-memory workspace requested for an axis that spans hosts")
        if nbytes <= self.sym_bytes and self.sym_ptrs:
            return
        size = max(int(nbytes) * 5 // 4, 1 << 21)
        size = (size + (1 << 21) - 1) >> 21 << 21
        _device_sync()
        dist.barrier(group=self.group)
        self._release_symmetric()
        C = _C()
        if not backend.emulated and NVLS:
            try:
                import torch.distributed._symmetric_memory as sm

                dev = torch.device("cuda", torch.cuda.current_device())
                t = sm.empty(size, dtype=torch.uint8, device=dev)
                h = sm.rendezvous(t, self.group.group_name)
                self._sym_tensor = t
                self.sym_ptrs = [int(p) for p in h.buffer_ptrs]
                self.sym_mc = int(h.multicast_ptr or 0)
            except Exception as e:  # allocator or fabric refused: the plain peer-memory form below
                self._sym_tensor, self.sym_ptrs, self.sym_mc = None, [], 0
                self.sym_error = repr(e)
            # every rank must take the same route
            ok = torch.tensor([1 if self.sym_ptrs else 0, 1 if self.sym_mc else 0], dtype=torch.int32,
                              device=torch.device("cuda", torch.cuda.current_device()))
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            ok = ok.tolist()
            if not ok[0]:
                self._sym_tensor, self.sym_ptrs, self.sym_mc = None, [], 0
            elif not ok[1]:
                self.sym_mc = 0
        if not self.sym_ptrs:
            dev = (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl"
                   else torch.device("cpu"))
            ptr, handle = C.symm_alloc(size)
            mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8).to(dev)
            allh = torch.empty(self.p * 64, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(allh, mine, group=self.group)
            allh = allh.cpu().view(self.p, 64)
            self.sym_ptrs = [ptr if q == self.rank else C.symm_open(bytes(allh[q].tolist())) for q in range(self.p)]
            self._sym_local, self.sym_mc = ptr, 0
        self.sym_bytes = size
        self.ensure(0)  # the flags
        _device_sync()
        dist.barrier(group=self.group)

    def _release_symmetric(self) -> None:
        if not self.sym_ptrs:
            return
        if self._sym_tensor is None:
            C = _C()
            for q, ptr in enumerate(self.sym_ptrs):
                if q != self.rank:
                    C.symm_close(ptr)
            try:
                dist.barrier(group=self.group)
            except Exception:
                pass
            C.symm_free(self._sym_local)
        self._sym_tensor, self._sym_local = None, 0
        self.sym_ptrs, self.sym_mc, self.sym_bytes = [], 0, 0

    def symmetric_view(self, rows: int, cols: int, dtype: torch.dtype, byte_off: int = 0) -> torch.Tensor:
        """``[rows, cols]`` tensor over this rank's symmetric buffer, ``byte_off`` bytes in."""
        esz = torch.empty(0, dtype=dtype).element_size()
        n = rows * cols
        if byte_off + n * esz > self.sym_bytes:
            raise ValueError("symmetric buffer too small")
        if self._sym_tensor is not None:
            return self._sym_tensor[byte_off : byte_off + n * esz].view(dtype).view(rows, cols)
        return _C().symm_view(self.sym_ptrs[self.rank] + byte_off, n, dtype).view(rows, cols)

    # -- addressing ---------------------------------------------------------------------
    def slot(self, owner: int, buf: int, src: int) -> int:
        """Address (in this process) of receive slot ``src`` of buffer ``buf`` on rank ``owner``."""
        return self.ptrs[owner] + FLAG_BYTES + (buf * self.p + src) * self.slot_bytes

    def flag(self, owner: int, buf: int, src: int) -> int:
        return self.ptrs[owner] + (buf * MAX_GROUP + src) * 4

    def next_op(self):
        self.epoch += 1
        return self.epoch, self.epoch % 2

    # -- sentinel buffers (all-reduces finished inside the compute kernels) --------------
    def sslot(self, owner: int, buf: int, src: int) -> int:
        base = self.ptrs[owner] + FLAG_BYTES + 2 * self.p * self.slot_bytes
        return base + (buf * self.p + src) * self.sslot_bytes

    def spush_targets(self, buf: int) -> List[int]:
        """This rank's sentinel slot in every peer's buffer."""
        out = PushList(self.sslot(q, buf, self.rank) for q in self.peers)
        out.limit_bytes = self.sslot_bytes if DEBUG else 0
        return out

    def tile_reduce(self, buf: int):
        """Argument tuple of the in-kernel all-reduce (see ``ops.cuda.gemm`` / ``ops.cuda.spmm``):
        every peer's sentinel slot in this rank's buffer, this rank's position, the wait limit."""
        return ([self.sslot(self.rank, buf, q) for q in self.peers], self.rank, self.timeout_ms)

    def push_targets(self, buf: int) -> List[int]:
        """This rank's slot in every peer's buffer."""
        out = PushList(self.slot(q, buf, self.rank) for q in self.peers)
        out.limit_bytes = self.slot_bytes if DEBUG else 0
        return out

    def recv_slots(self, buf: int) -> List[int]:
        """Every peer's slot in this rank's buffer."""
        return [self.slot(self.rank, buf, q) for q in self.peers]

    def sync(self, buf: int):
        remote = [self.flag(q, buf, self.rank) for q in self.peers]
        local = [self.flag(self.rank, buf, q) for q in self.peers]
        return remote, local


_axes: Dict[tuple, AxisComm] = {}


def axis_for(group, channel: int = 0) -> AxisComm:
    """The workspace of ``group``.  A *channel* is an independent workspace (own flags, buffers and op
    counter) on the same group: ops of one channel must be issued and executed in the same order on
    every rank, so traffic that runs on another stream (the weight-gradient reductions) gets its own."""
    key = (id(group), channel)
    if key not in _axes:
        _axes[key] = AxisComm(group)
    return _axes[key]


def setup(grid) -> None:
    """Create the (empty) workspace objects of this rank's three line groups."""
    for axis in ("x", "y", "z"):
        g = grid.group(axis)
        if g is not None:
            axis_for(g)


def teardown() -> None:
    if _axes:
        _device_sync()
    for ax in _axes.values():
        try:
            ax._release_symmetric()
            ax.release()
        except Exception:
            pass
    _axes.clear()
