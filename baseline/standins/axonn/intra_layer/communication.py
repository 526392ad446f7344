"""Collective wrappers with the call signatures plexus/gcn_conv.py uses."""

import torch
import torch.distributed as dist

from axonn import axonn as ax


def _all_reduce(input_, process_group=None):
    if dist.get_world_size(process_group) == 1:
        return input_
    ax.get_timers.start("all-reduce")
    dist.all_reduce(input_.contiguous(), group=process_group)
    ax.get_timers.stop("all-reduce")
    return input_


def _gather(input_, dim, process_group=None):
    p = dist.get_world_size(process_group)
    if p == 1:
        return input_
    ax.get_timers.start("gather")
    input_ = input_.contiguous()
    parts = [torch.empty_like(input_) for _ in range(p)]
    dist.all_gather(parts, input_, group=process_group)
    out = torch.cat(parts, dim=dim).contiguous()
    ax.get_timers.stop("gather")
    return out


def _reduce_scatter(input_, dim, process_group=None):
    assert dim == 0
    p = dist.get_world_size(process_group)
    if p == 1:
        return input_
    ax.get_timers.start("reduce-scatter")
    assert input_.shape[0] % p == 0
    out = torch.empty((input_.shape[0] // p,) + tuple(input_.shape[1:]), dtype=input_.dtype,
                      device=input_.device)
    dist.reduce_scatter_tensor(out, input_.contiguous(), group=process_group)
    ax.get_timers.stop("reduce-scatter")
    return out
