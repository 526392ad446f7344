"""Class-sharded softmax cross-entropy for logits laid out ``(N/rows) x (C/classes)``.

The logits of an ``L``-layer GCN are sharded by rows over the depth axis and by
classes over the outer axis of the last layer.  The loss is

    sum over valid rows of  -log softmax(logits)[label]  /  num_nodes

where a row is valid if it is a real node (not padding) and its label is
non-negative.  Per row, each class shard contributes ``(max, sum exp)``; the
pairs of all class shards are exchanged once over the class axis (an all-gather
of ``2 x rows`` floats, through peer memory in fused mode) and combined locally;
the scalar loss is summed over both axes.  The reference issues three
class-axis all-reduces of ``rows`` floats (plexus/cross_entropy.py:46-92).

Reference: plexus/cross_entropy.py:13-120.  Unlike the reference this
implementation never writes into ``logits`` or ``target``, stores neither a
softmax nor a one-hot matrix (backward recomputes the probabilities from the
logits and the two row statistics), and gives padded rows no loss.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops, runtime
from ..parallel import collectives as coll
from ..parallel.grid import get_grid, group_size, loss_axes
from ..utils.timers import get_timers


class TensorParallelCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, num_layers, num_nodes, num_classes, row_weight=None):
        timers = get_timers()
        timers.start("cross entropy fwd")
        grid = get_grid()
        row_axis, class_axis = loss_axes(num_layers)
        row_group, class_group = grid.group(row_axis), grid.group(class_axis)
        row_offset = grid.coord(row_axis) * logits.shape[0]
        class_offset = grid.coord(class_axis) * logits.shape[1]

        logits = logits.contiguous()
        if group_size(class_group) > 1:
            # one exchange over the class axis: every shard's (max, sum exp) pair per row; one kernel
            # combines them in rank order (so all class shards hold bitwise identical statistics)
            # and adds up the loss terms of the local targets
            res = None
            if runtime.flags.comm == "fused" and not runtime.flags.skip_collectives:
                from ..parallel import fused

                if fused.XENT_EXCHANGE:
                    # the two kernels exchange the pairs themselves (push + flagged read)
                    res = fused.xent_exchange_combine(logits, target, class_offset, num_classes, row_offset,
                                                      num_nodes, row_weight, class_group)
            if res is None:
                stats, _ = ops.xent_stats(logits, class_offset, num_classes)
                pairs = coll.all_gather(stats.unsqueeze(0), dim=0, process_group=class_group)
                res = ops.xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, row_weight)
            stats, loss = res
        else:
            # classes not sharded: statistics and loss in one pass over the logits
            stats, loss = ops.xent_stats(logits, class_offset, num_classes, target, row_offset, num_nodes,
                                         row_weight)
        gmax, gsum = stats[0], stats[1]
        loss = loss.reshape(1)
        # one scalar reduction over both axes (class shards hold disjoint terms)
        coll.all_reduce(loss, class_group)
        coll.all_reduce(loss, row_group)
        loss = (loss / num_nodes).reshape(())

        ctx.save_for_backward(logits, target, gmax, gsum)
        ctx.meta = (row_offset, class_offset, num_nodes, num_classes)
        ctx.row_weight = row_weight
        timers.stop("cross entropy fwd")
        return loss

    @staticmethod
    def backward(ctx, grad_output):
        timers = get_timers()
        timers.start("cross entropy bwd")
        logits, target, gmax, gsum = ctx.saved_tensors
        row_offset, class_offset, num_nodes, num_classes = ctx.meta
        grad = ops.xent_grad(
            logits, target, gmax, gsum, row_offset, class_offset, num_nodes, num_classes,
            grad_output / num_nodes,
        )
        if ctx.row_weight is not None:
            grad = grad * ctx.row_weight.unsqueeze(1).to(grad.dtype)
        timers.stop("cross entropy bwd")
        return grad, None, None, None, None, None


def parallel_cross_entropy(logits, target, num_layers, num_nodes, num_classes, row_weight=None):
    """Mean (over ``num_nodes``) cross-entropy of class-sharded logits.

    ``num_layers`` selects which grid axes shard the rows and the classes.
    ``row_weight`` (optional 0/1 or real weights per local row) restricts the
    loss, e.g. to a training mask.
    """
    return TensorParallelCrossEntropy.apply(
        logits, target, num_layers, num_nodes, num_classes, row_weight
    )


def parallel_accuracy(logits, target, num_layers, num_nodes, num_classes, mask=None):
    """Fraction of valid (optionally masked) rows whose arg-max class equals the label."""
    grid = get_grid()
    row_axis, class_axis = loss_axes(num_layers)
    row_group, class_group = grid.group(row_axis), grid.group(class_axis)
    R, C = logits.shape
    class_offset = grid.coord(class_axis) * C
    row_offset = grid.coord(row_axis) * R
    cls = torch.arange(C, device=logits.device) + class_offset
    lf = logits.detach().float().masked_fill((cls >= num_classes).unsqueeze(0), float("-inf"))
    lmax, larg = lf.max(dim=1)
    gmax = lmax.clone()
    coll.all_reduce(gmax, class_group, op=dist.ReduceOp.MAX)
    # smallest global class index attaining the max
    cand = torch.where(lmax == gmax, larg + class_offset, torch.full_like(larg, num_classes))
    cand = cand.to(torch.float32)
    coll.all_reduce(cand, class_group, op=dist.ReduceOp.MIN)
    rows = torch.arange(R, device=logits.device) + row_offset
    valid = (rows < num_nodes) & (target >= 0)
    if mask is not None:
        valid = valid & mask
    stats = torch.stack([((cand.long() == target) & valid).sum(), valid.sum()]).to(torch.float64)
    coll.all_reduce(stats, row_group)
    return (stats[0] / stats[1].clamp(min=1)).item()
