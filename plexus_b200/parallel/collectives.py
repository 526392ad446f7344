"""Library-path collectives over ``torch.distributed`` (NCCL on GPU, gloo on CPU).

These are the unfused versions of the collectives a 3D-parallel GCN layer
needs: depth-axis all-gather, in-place SUM all-reduce and reduce-scatter.  A
``None`` group (an axis of size 1) makes every call a no-op.  Each call is
wrapped in a timer region named ``gather`` / ``all-reduce`` /
``reduce-scatter`` so a log parser can sum the communication time
(reference: examples/parse_results.py:46-54; the wrappers replace AxoNN's
``_gather``, ``_all_reduce`` and ``_reduce_scatter`` used at
plexus/gcn_conv.py:177-278).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import runtime
from ..utils.timers import get_timers
from .grid import group_size


def _fused(t: torch.Tensor) -> bool:
    if runtime.flags.comm != "fused":
        return False
    if t.is_cuda:
        return True
    from . import backend

    return backend.emulated

_bytes_moved = {"gather": 0, "all-reduce": 0, "reduce-scatter": 0}


def bytes_moved(reset: bool = False):
    """Payload bytes handed to each collective kind since the last reset."""
    out = dict(_bytes_moved)
    if reset:
        for k in _bytes_moved:
            _bytes_moved[k] = 0
    return out


def all_gather(t: torch.Tensor, dim: int = 0, process_group=None) -> torch.Tensor:
    """Concatenate every rank's ``t`` along ``dim`` (rank order)."""
    p = group_size(process_group)
    if p == 1:
        return t
    if runtime.flags.skip_collectives:
        reps = [1] * t.dim()
        reps[dim] = p
        return t.repeat(*reps)
    timers = get_timers()
    timers.start("gather")
    t = t.contiguous()
    _bytes_moved["gather"] += t.numel() * t.element_size() * (p - 1)
    if dim == 0 and _fused(t) and (t.numel() * t.element_size()) % 4 == 0:
        from . import fused

        out = fused.all_gather(t, process_group)
    elif dim == 0:
        out = torch.empty((p * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=process_group)
    else:
        parts = torch.empty((p,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(parts, t, group=process_group)
        out = torch.cat(list(parts.unbind(0)), dim=dim)
    timers.stop("gather")
    return out


def all_reduce(t: torch.Tensor, process_group=None, op=None) -> torch.Tensor:
    """In-place SUM (or ``op``) all-reduce; returns ``t``."""
    if group_size(process_group) == 1 or runtime.flags.skip_collectives:
        return t
    timers = get_timers()
    timers.start("all-reduce")
    _bytes_moved["all-reduce"] += t.numel() * t.element_size()
    if _fused(t) and op in (None, dist.ReduceOp.SUM, dist.ReduceOp.MAX):
        from . import fused

        if fused.supports(t) and (t.dtype == torch.float32 or op in (None, dist.ReduceOp.SUM)):
            if t.dtype == torch.float32:
                fused.all_reduce_f32(t, process_group, op)
            else:
                fused.all_reduce_bf16(t, process_group)
            timers.stop("all-reduce")
            return t
    if not t.is_contiguous():
        tmp = t.contiguous()
        dist.all_reduce(tmp, op=op or dist.ReduceOp.SUM, group=process_group)
        t.copy_(tmp)
    else:
        dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=process_group)
    timers.stop("all-reduce")
    return t


def reduce_scatter(t: torch.Tensor, dim: int = 0, process_group=None) -> torch.Tensor:
    """SUM-reduce ``t`` over the group and return this rank's 1/p slice along ``dim``."""
    p = group_size(process_group)
    if p == 1:
        return t
    if dim != 0:
        raise NotImplementedError("reduce_scatter is only used along dim 0")
    if t.shape[0] % p != 0:
        raise ValueError(f"reduce_scatter: leading size {t.shape[0]} not divisible by {p}")
    if runtime.flags.skip_collectives:
        return t[: t.shape[0] // p].clone()
    timers = get_timers()
    timers.start("reduce-scatter")
    t = t.contiguous()
    _bytes_moved["reduce-scatter"] += t.numel() * t.element_size()
    out = torch.empty((t.shape[0] // p,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if _fused(t):
        from . import fused

        if fused.supports(t):
            # peer-memory all-reduce of a copy, then keep this rank's slice
            tmp = t.clone()
            if tmp.dtype == torch.float32:
                fused.all_reduce_f32(tmp, process_group)
            else:
                fused.all_reduce_bf16(tmp.view(-1, 8) if tmp.dim() == 1 and tmp.numel() % 8 == 0 else tmp,
                                      process_group)
            r = dist.get_rank(process_group)
            out.copy_(tmp[r * out.shape[0] : (r + 1) * out.shape[0]])
            timers.stop("reduce-scatter")
            return out
    if t.device.type == "cpu":
        # gloo has no reduce_scatter_tensor: all-reduce a copy and slice.
        tmp = t.clone()
        dist.all_reduce(tmp, group=process_group)
        r = dist.get_rank(process_group)
        out.copy_(tmp[r * out.shape[0] : (r + 1) * out.shape[0]])
    else:
        dist.reduce_scatter_tensor(out, t, group=process_group)
    timers.stop("reduce-scatter")
    return out


class PendingReduce:
    """Result of a reduction that may still be in flight; ``wait()`` returns the tensor."""

    def __init__(self, result: torch.Tensor, work=None, finish=None):
        self._result, self._work, self._finish = result, work, finish

    def wait(self) -> torch.Tensor:
        if self._work is not None:
            self._work.wait()  # the current stream waits for the collective's stream
            self._work = None
        if self._finish is not None:
            self._result = self._finish(self._result)
            self._finish = None
        return self._result


def reduce_grad_async(t: torch.Tensor, process_group=None, scatter: bool = False) -> PendingReduce:
    """Start ``all_reduce`` (or, with ``scatter``, ``reduce_scatter`` along dim 0) of a gradient.

    On the library path the collective is issued asynchronously on the communicator's own stream,
    so the kernels launched before ``wait()`` (the rest of a layer's backward) overlap it; the
    weight gradient is not needed before the optimizer step.  The peer-memory path and
    single-rank groups complete immediately.
    """
    p = group_size(process_group)
    if p == 1:
        return PendingReduce(t)
    if runtime.flags.skip_collectives:
        return PendingReduce(reduce_scatter(t, 0, process_group) if scatter else t)
    if _fused(t) and t.is_contiguous() and (t.dtype == torch.float32 or not t.is_cuda):
        from . import fused

        ax_ok = fused.symm.axis_for(process_group, fused.GRAD_CHANNEL).same_host
        small = t.numel() * t.element_size() <= fused.SMALL_MESSAGE_BYTES or p <= fused.ONE_SHOT_MAX_RANKS
        if ax_ok and small and fused.supports(t) and (not scatter or t.shape[0] % p == 0):
            # peer-memory kernels on their own workspace channel and (untimed runs) a side stream
            kind = "reduce-scatter" if scatter else "all-reduce"
            _bytes_moved[kind] += t.numel() * t.element_size()
            timed = get_timers().enabled
            if timed:
                get_timers().start(kind)
            result, join = fused.reduce_grad_f32(t, process_group, scatter, overlap=not timed)
            if timed:
                get_timers().stop(kind)
            return PendingReduce(result, finish=lambda r, _j=join: (_j(), r)[1])
    if _fused(t) or t.device.type == "cpu" or get_timers().enabled:
        # in-line: peer-memory kernels are stream-ordered already; timed runs keep the
        # collective inside its own timer region
        return PendingReduce(reduce_scatter(t, 0, process_group) if scatter else all_reduce(t, process_group))
    t = t.contiguous()
    if scatter:
        if t.shape[0] % p != 0:
            raise ValueError(f"reduce_scatter: leading size {t.shape[0]} not divisible by {p}")
        _bytes_moved["reduce-scatter"] += t.numel() * t.element_size()
        out = torch.empty((t.shape[0] // p,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        work = dist.reduce_scatter_tensor(out, t, group=process_group, async_op=True)
        # keep the input alive until the collective has consumed it
        return PendingReduce(out, work, finish=lambda r, _keep=t: r)
    _bytes_moved["all-reduce"] += t.numel() * t.element_size()
    work = dist.all_reduce(t, group=process_group, async_op=True)
    return PendingReduce(t, work)


# Names used by code written against AxoNN's intra-layer communication module.
_gather = all_gather
_all_reduce = all_reduce
_reduce_scatter = reduce_scatter
