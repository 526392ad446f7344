"""Op dispatch: CUDA tensors go to the sm_100a kernels, CPU tensors to torch.

There is exactly one GPU implementation of each op (the hand-written kernels
in ``plexus_b200/csrc``); the torch versions in :mod:`.reference` serve CPU
runs (gloo plumbing, serial oracle) and tests.  If the compiled extension is
missing on a machine with a GPU the first CUDA call raises.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import reference

extract_csr_submatrix = reference.extract_csr_submatrix


def _cuda():
    from . import cuda as _c

    return _c


def spmm(A, H, relu_mask=None, row_range: Optional[Tuple[int, int]] = None, out_dtype=None, out=None):
    """``A[row_range] @ H`` (fp32 accumulate), optionally masked by ``relu_mask > 0``."""
    if H.is_cuda:
        return _cuda().spmm(A, H, relu_mask=relu_mask, row_range=row_range, out_dtype=out_dtype, out=out)
    res = reference.spmm(A, H, relu_mask=relu_mask, row_range=row_range, out_dtype=out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def gemm(a, b, trans_a=False, trans_b=False, relu=False, out_dtype=None, relu_mask=None):
    """``op(a) @ op(b)`` (fp32 accumulate) with optional fused ReLU or ``* (relu_mask > 0)``."""
    if a.is_cuda and not trans_a:
        return _cuda().gemm(a, b, trans_a=trans_a, trans_b=trans_b, relu=relu, out_dtype=out_dtype,
                            relu_mask=relu_mask)
    if a.is_cuda:
        out = _cuda().gemm(a, b, trans_a=trans_a, trans_b=trans_b, relu=relu, out_dtype=out_dtype)
    else:
        out = reference.gemm(a, b, trans_a=trans_a, trans_b=trans_b, relu=relu, out_dtype=out_dtype)
    return out if relu_mask is None else relu_backward(out, relu_mask)


def relu_backward(grad, out):
    if grad.is_cuda:
        return _cuda().relu_backward(grad, out)
    return reference.relu_backward(grad, out)


def xent_local_stats(logits, class_offset, num_classes):
    if logits.is_cuda:
        return _cuda().xent_local_stats(logits, class_offset, num_classes)
    return reference.xent_local_stats(logits, class_offset, num_classes)


def xent_stats(logits, class_offset, num_classes, target=None, row_offset=0, num_nodes=0, weight=None):
    """``(stats [2, R], loss or None)``: per-row (max, sum exp) of this class shard; with ``target``
    (classes not sharded) the loss comes out of the same pass."""
    mod = _cuda() if logits.is_cuda else reference
    return mod.xent_stats(logits, class_offset, num_classes, target, row_offset, num_nodes, weight)


def xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, weight=None):
    """``pairs [P, 2, R]`` of all class shards -> ``(stats [2, R], loss)`` in one pass."""
    mod = _cuda() if logits.is_cuda else reference
    return mod.xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, weight)


def xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, weight=None):
    if logits.is_cuda:
        return _cuda().xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, weight)
    return reference.xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, weight)


def xent_grad(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, num_classes, scale,
              out_dtype=None):
    if logits.is_cuda:
        return _cuda().xent_grad(logits, target, gmax, gsum, row_offset, class_offset, num_nodes,
                                 num_classes, scale, out_dtype)
    return reference.xent_grad(logits, target, gmax, gsum, row_offset, class_offset, num_nodes,
                               num_classes, scale, out_dtype)
