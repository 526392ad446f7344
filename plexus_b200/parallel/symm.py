"""Symmetric peer-memory workspaces, one per grid axis this rank belongs to.

A workspace is one ``cudaMalloc`` per rank whose CUDA-IPC handle is exchanged over the axis'
process group, so every rank holds a device pointer into every peer's buffer and kernels can
store into / load from peer memory directly over NVLink.  Layout of each rank's buffer::

    [ flags: int32[2][8] (1 KiB) | signals: int32[2][8][SIG_INTS] | buffer 0: p slots | buffer 1: p slots ]

The signals serve the kernels that finish an all-reduce themselves: per (buffer, source rank) the
first ``GEMM_SIG_INTS`` entries are written by the source's GEMM CTAs (one entry per CTA, counting
the tiles it has pushed), the next ``TILE_SIG_INTS`` count, per fixed block of output rows, how
many rows of that block the source's SpMM has pushed.

Slot ``s`` of a buffer receives data from group rank ``s``.  The op counter ("epoch") of an axis
selects buffer ``epoch % 2``; see ``csrc/kernels/comm_fused.cu`` for the flag protocol and why
double buffering is enough.  Workspaces grow on demand (a collective operation: every rank of
the axis asks for the same size at the same point of the program).
"""

from __future__ import annotations

import hashlib
import os
import socket
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _ext
from . import emulator


def _C():
    """The extension, or its host emulation when that is enabled (CPU ranks, tests)."""
    return emulator.C if emulator.active() else _ext.load()


def _device_sync() -> None:
    if not emulator.active():
        torch.cuda.synchronize()

MAX_GROUP = 8
OP_FLAG_BYTES = 1024
GEMM_SIG_INTS = 256          # >= the largest grid of the tcgen05 GEMM
TILE_SIG_INTS = 65536        # row blocks of one SpMM output
SIG_INTS = GEMM_SIG_INTS + TILE_SIG_INTS
FLAG_BYTES = OP_FLAG_BYTES + 2 * MAX_GROUP * SIG_INTS * 4
EPOCH_LIMIT = 100000         # signal values are epoch << 14 + count: stay far below 2^31
DEFAULT_TIMEOUT_MS = 5000.0


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
        self.local_ptr = 0
        self.ptrs: List[int] = []
        self.timeout_ms = DEFAULT_TIMEOUT_MS
        self._local_done = None  # per-tile row counters of this rank's own SpMM (device-local)

    # -- allocation ---------------------------------------------------------------------
    def ensure(self, slot_bytes: int) -> None:
        if not self.same_host:
            raise RuntimeError("peer-memory workspace requested for an axis that spans hosts")
        slot_bytes = (int(slot_bytes) + 1023) // 1024 * 1024
        if slot_bytes <= self.slot_bytes:
            return
        C = _C()
        dev = (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl"
               else torch.device("cpu"))
        # nobody may still be using the old workspace
        _device_sync()
        dist.barrier(group=self.group)
        self.release()
        total = FLAG_BYTES + 2 * self.p * slot_bytes
        ptr, handle = C.symm_alloc(total)
        mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8).to(dev)
        allh = torch.empty(self.p * 64, dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allh, mine, group=self.group)
        allh = allh.cpu().view(self.p, 64)
        self.ptrs = []
        for q in range(self.p):
            self.ptrs.append(ptr if q == self.rank else C.symm_open(bytes(allh[q].tolist())))
        self.local_ptr, self.slot_bytes = ptr, slot_bytes
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
        self.ptrs, self.local_ptr, self.slot_bytes = [], 0, 0

    # -- addressing ---------------------------------------------------------------------
    def slot(self, owner: int, buf: int, src: int) -> int:
        """Address (in this process) of receive slot ``src`` of buffer ``buf`` on rank ``owner``."""
        return self.ptrs[owner] + FLAG_BYTES + (buf * self.p + src) * self.slot_bytes

    def flag(self, owner: int, buf: int, src: int) -> int:
        return self.ptrs[owner] + (buf * MAX_GROUP + src) * 4

    def next_op(self):
        if self.epoch >= EPOCH_LIMIT:
            self._restart_epochs()
        self.epoch += 1
        return self.epoch, self.epoch % 2

    def _restart_epochs(self) -> None:
        """Start counting ops from zero again (collective: every rank of the axis reaches the limit
        at the same op).  Nobody may still be waiting on an old value when the flags are cleared."""
        _device_sync()
        dist.barrier(group=self.group)
        _C().symm_clear(self.local_ptr, FLAG_BYTES)
        _device_sync()
        dist.barrier(group=self.group)
        self.epoch = 0

    def sig_base(self, epoch: int) -> int:
        return epoch << 14

    def gemm_sig(self, owner: int, buf: int, src: int) -> int:
        """Address of the per-CTA signal array that rank ``src`` writes inside ``owner``'s workspace."""
        return self.ptrs[owner] + OP_FLAG_BYTES + ((buf * MAX_GROUP + src) * SIG_INTS) * 4

    def tile_sig(self, owner: int, buf: int, src: int) -> int:
        """Address of the per-row-block counters that rank ``src`` adds to inside ``owner``'s workspace."""
        return self.gemm_sig(owner, buf, src) + GEMM_SIG_INTS * 4

    def tile_reduce_gemm(self, epoch: int, buf: int):
        """Argument tuple of the GEMM's in-kernel all-reduce for op ``epoch`` (see ``ops.cuda.gemm``)."""
        return (self.recv_slots(buf), [self.gemm_sig(q, buf, self.rank) for q in self.peers],
                [self.gemm_sig(self.rank, buf, q) for q in self.peers], self.sig_base(epoch), self.rank,
                self.timeout_ms)

    def tile_reduce_spmm(self, buf: int, out_rows: int):
        """Argument tuple of the SpMM's in-kernel all-reduce (see ``ops.cuda.spmm``): exchange tiles of
        at least 512 output rows, at most ``TILE_SIG_INTS`` of them."""
        tile_rows = max(512, -(-out_rows // TILE_SIG_INTS))
        tile_rows = -(-tile_rows // 128) * 128
        if self._local_done is None:
            dev = "cpu" if emulator.active() else torch.device("cuda", torch.cuda.current_device())
            self._local_done = torch.zeros(TILE_SIG_INTS, dtype=torch.int32, device=dev)
        return (self.recv_slots(buf), [self.tile_sig(q, buf, self.rank) for q in self.peers],
                [self.tile_sig(self.rank, buf, q) for q in self.peers], self.rank, self.timeout_ms, tile_rows,
                self._local_done.data_ptr())

    def push_targets(self, buf: int) -> List[int]:
        """This rank's slot in every peer's buffer."""
        return [self.slot(q, buf, self.rank) for q in self.peers]

    def recv_slots(self, buf: int) -> List[int]:
        """Every peer's slot in this rank's buffer."""
        return [self.slot(self.rank, buf, q) for q in self.peers]

    def sync(self, buf: int):
        remote = [self.flag(q, buf, self.rank) for q in self.peers]
        local = [self.flag(self.rank, buf, q) for q in self.peers]
        return remote, local


_axes: Dict[int, AxisComm] = {}


def axis_for(group) -> AxisComm:
    key = id(group)
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
            ax.release()
        except Exception:
            pass
    _axes.clear()
