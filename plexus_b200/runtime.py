"""Framework initialisation and run-time flags.

``init`` keeps the keyword signature of the reference's ``plexus.init``
(reference: plexus/plexus.py:5-48) and adds B200-specific switches:

* ``comm``: ``"nccl"`` issues every collective through ``torch.distributed``
  (the library path, also the only one on CPU/gloo); ``"fused"`` routes the
  aggregation / combination collectives through kernels that read and write
  peer memory over NVLink (see ``plexus_b200.parallel.symm``).
* ``dtype``: storage type of features, activations and their gradients on the
  device (accumulation is always fp32).  ``None`` picks bf16 on CUDA and fp32
  on CPU.
* ``channel_align``: local channel counts are padded to a multiple of this
  many elements so that every feature row starts on a 16-byte boundary
  (needed by vector loads and TMA).  ``None`` picks 8 on CUDA, 1 on CPU.
* ``grid="auto"``: ask the performance models for the grid shape.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .parallel import grid as _grid
from .utils import timers as _timers


@dataclass
class Flags:
    block_agg: bool = False
    overlap_agg: bool = False
    tune_gemm: bool = False
    comm: str = "nccl"
    dtype: torch.dtype = torch.float32
    channel_align: int = 1
    initialized: bool = False
    # measurement aid: every collective becomes a local stand-in of the same shapes (results are
    # then wrong); epoch time with it on = compute-only time of the same shards, and
    # "exposed communication" = normal epoch time minus that
    skip_collectives: bool = False


flags = Flags()

# Module-level mirrors, read directly by code written against the reference
# (``plx.block_agg`` etc., reference: plexus/plexus.py:43-48).
block_agg = False
overlap_agg = False
tune_gemm = False


def init(
    G_intra_r: int = 1,
    G_intra_c: int = 1,
    G_intra_d: int = 1,
    gpus_per_node: Optional[int] = None,
    enable_internal_timers: bool = False,
    block_aggregation: bool = False,
    overlap_aggregation: bool = False,
    tune_gemms: bool = False,
    *,
    comm: Optional[str] = None,
    dtype: Optional[torch.dtype] = None,
    channel_align: Optional[int] = None,
    device: Optional[str] = None,
) -> _grid.ProcessGrid:
    """Set up the X x Y x Z grid (X=G_intra_r, Y=G_intra_c, Z=G_intra_d).

    ``torch.distributed`` must already be initialised when the grid has more
    than one rank.  Returns the :class:`ProcessGrid`.
    """
    global block_agg, overlap_agg, tune_gemm

    # Overlapping the aggregation all-reduce only makes sense on row blocks.
    assert not overlap_aggregation or block_aggregation, (
        "overlap_aggregation requires block_aggregation"
    )

    use_cuda = torch.cuda.is_available() and device != "cpu"
    if use_cuda:
        if gpus_per_node is None:
            gpus_per_node = torch.cuda.device_count()
        rank = dist.get_rank() if dist.is_initialized() else 0
        torch.cuda.set_device(rank % max(1, gpus_per_node))

    g = _grid.ProcessGrid.build(G_intra_r, G_intra_c, G_intra_d)
    _grid.set_grid(g)

    _timers.configure_timers(enable_internal_timers, use_cuda=use_cuda)

    flags.block_agg = block_agg = bool(block_aggregation)
    flags.overlap_agg = overlap_agg = bool(overlap_aggregation)
    flags.tune_gemm = tune_gemm = bool(tune_gemms)
    flags.comm = comm if comm is not None else "nccl"
    if flags.comm not in ("nccl", "fused"):
        raise ValueError("comm must be 'nccl' or 'fused'")
    from .parallel import backend, emulator

    if flags.comm == "fused" and not use_cuda and not emulator.active():
        raise ValueError("comm='fused' needs CUDA devices with peer access "
                         "(or parallel.emulator.enable() to emulate them on CPU ranks)")
    # the kernels behind the peer-memory collectives are chosen here, once
    backend.bind(flags.comm == "fused" and emulator.active())
    if use_cuda and dtype not in (None, torch.bfloat16):
        raise ValueError("on CUDA devices the model runs in bf16 (fp32 accumulation, fp32 master weights): the "
                         "tcgen05 GEMMs take bf16 operands only; dtype=torch.float32 is for CPU runs")
    flags.dtype = dtype if dtype is not None else (torch.bfloat16 if use_cuda else torch.float32)
    flags.channel_align = (
        channel_align if channel_align is not None else (8 if use_cuda else 1)
    )
    flags.initialized = True

    if flags.comm == "fused" and g.world_size > 1:
        from .parallel import symm

        symm.setup(g)
    return g


def check_status() -> None:
    """Raise :class:`plexus_b200.parallel.watchdog.PlexusCommTimeout` if a kernel's bounded wait (on a
    peer's flag, or on one of its own asynchronous copies) gave up since the last check.

    Such a kernel returns without producing its result, so everything computed after it in the step
    is garbage: call this after each step (it synchronises the device) and before anything derived
    from the step is persisted - a checkpoint above all.
    """
    if flags.comm == "fused":
        from .parallel import backend

        if backend.emulated:
            backend.ops().check_status()
            return
    if torch.cuda.is_available():
        from .ops import cuda as _opc

        _opc.check_status()


def inject_status_timeout(kernel_id: int = 99) -> None:
    """Host-side fault injection: write the record a kernel leaves when a bounded wait runs out
    (``TIMEOUT, kernel, peer, expected, seen``) into the status words, without running any kernel."""
    from .parallel.watchdog import STATUS_TIMEOUT

    rec = torch.tensor([STATUS_TIMEOUT, kernel_id, 0, 1, 0], dtype=torch.int32)
    if flags.comm == "fused":
        from .parallel import backend

        if backend.emulated:
            backend.ops().status_buffer()[:5] = rec
            return
    if torch.cuda.is_available():
        from .ops import cuda as _opc

        _opc.status_buffer()[:5] = rec.to(_opc.status_buffer().device)
        return
    raise RuntimeError("no status words on this path (CPU ranks without the peer-memory emulation)")


def shutdown() -> None:
    """Forget the grid (process groups are left to ``destroy_process_group``)."""
    if flags.comm == "fused":
        from .parallel import symm

        symm.teardown()
    _grid.set_grid(None)
    flags.initialized = False


def choose_grid(world_size: int, num_nodes: int, num_nonzeros: int, dims, machine="b200_nvl8"):
    """Grid shape (X, Y, Z) the cost models rank first for this graph."""
    from .perf.chooser import choose_grid as _choose

    return _choose(world_size, num_nodes, num_nonzeros, list(dims), machine=machine)[0]
