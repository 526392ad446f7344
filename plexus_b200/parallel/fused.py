"""Collectives carried out by kernels that store into / load from peer memory over NVLink.

* ``spmm_all_reduce`` / ``gemm_all_reduce``: the compute kernel's epilogue writes every result
  row to the local output *and* into this rank's receive slot on each peer of the axis (plain
  16-byte stores, overlapped with the rest of the kernel's work); a second launch publishes a
  flag, waits for the peers' flags and sums the received partials into the output in fp32
  (ReLU / ReLU-derivative mask applied after the sum).
* ``all_reduce_f32`` (SUM / MAX) and ``all_gather``: push-copy kernel + flagged consumer, used
  for the cross-entropy row statistics, weight shards and weight gradients.

These replace the NCCL calls of ``parallel.collectives`` when ``init(comm="fused")`` is used
(reference call sites: plexus/gcn_conv.py:177-278, plexus/cross_entropy.py:46-98).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops import cuda as opc
from . import symm

import os

KID_SPMM, KID_GEMM, KID_GATHER, KID_BARRIER, KID_XENT = 1, 2, 3, 4, 5

# The push epilogue is a one-shot all-reduce: every rank sends its whole partial result to every
# peer, (p-1) x M bytes per rank.  For p = 2 that is the minimum; measured on 4 GPUs it loses to
# NCCL's bandwidth-optimal ring (2 (p-1)/p x M), so larger groups reduce large messages with NCCL
# after the compute kernel.  Small messages (latency bound) always use the push path.
ONE_SHOT_MAX_RANKS = int(os.environ.get("PLEXUS_ONE_SHOT_MAX_RANKS", "2"))
SMALL_MESSAGE_BYTES = 1 << 20


def _push_path(ax, nbytes: int) -> bool:
    return ax.p <= ONE_SHOT_MAX_RANKS or nbytes <= SMALL_MESSAGE_BYTES


def _reduce(ax, out, buf, epoch, relu, mask, kid):
    remote, local = ax.sync(buf)
    _ext.load().reduce_slots(out, ax.recv_slots(buf), out.stride(0), bool(relu), mask, remote, local,
                             epoch, ax.timeout_ms, kid, opc.status_buffer(out.device))
    opc._count(1)


def spmm_all_reduce(A, H, group, relu_mask=None):
    """``all_reduce_sum(A @ H)`` over ``group`` with the push fused in the SpMM epilogue."""
    ax = symm.axis_for(group)
    rows, D = A.shape[0], H.shape[1]
    if not _push_path(ax, rows * D * H.element_size()):
        out = opc.spmm(A, H)
        dist.all_reduce(out, group=group)
        return out if relu_mask is None else opc.relu_backward(out, relu_mask)
    ax.ensure(rows * D * H.element_size())
    epoch, buf = ax.next_op()
    out = opc.spmm(A, H, push_ptrs=ax.push_targets(buf), push_ld=D)
    if relu_mask is not None and relu_mask.dtype != out.dtype:
        relu_mask = relu_mask.to(out.dtype)
    _reduce(ax, out, buf, epoch, False, relu_mask, KID_SPMM)
    return out


def gemm_all_reduce(a, W, group, relu=False, trans_b=False):
    """``act(all_reduce_sum(a @ op(W)))`` with the push fused in the tcgen05 GEMM epilogue."""
    ax = symm.axis_for(group)
    rows = a.shape[0]
    N = W.shape[0] if trans_b else W.shape[1]
    if not _push_path(ax, rows * N * a.element_size()):
        out = opc.gemm(a, W, trans_b=trans_b, relu=False)
        dist.all_reduce(out, group=group)
        return torch.relu_(out) if relu else out
    ax.ensure(rows * N * a.element_size())
    epoch, buf = ax.next_op()
    out = opc.gemm(a, W, trans_b=trans_b, relu=False, push_ptrs=ax.push_targets(buf), push_ld=N)
    _reduce(ax, out, buf, epoch, relu, None, KID_GEMM)
    return out


def all_reduce_f32(t: torch.Tensor, group, op=None) -> torch.Tensor:
    """In-place SUM or MAX all-reduce of a contiguous fp32 tensor."""
    if op in (None, dist.ReduceOp.SUM):
        code = 0
    elif op == dist.ReduceOp.MAX:
        code = 1
    else:
        raise NotImplementedError("fused all-reduce supports SUM and MAX")
    assert t.dtype == torch.float32 and t.is_contiguous()
    if t.numel() == 0:
        return t
    ax = symm.axis_for(group)
    C = _ext.load()
    if not _push_path(ax, t.numel() * 4):
        dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=group)
        return t
    ax.ensure(t.numel() * 4)
    epoch, buf = ax.next_op()
    C.push_copy(t, ax.push_targets(buf))
    remote, local = ax.sync(buf)
    C.reduce_slots_f32(t.view(-1), ax.recv_slots(buf), code, remote, local, epoch, ax.timeout_ms,
                       KID_XENT, opc.status_buffer(t.device))
    opc._count(2)
    return t


def all_gather(t: torch.Tensor, group) -> torch.Tensor:
    """Concatenate every rank's contiguous ``t`` along dim 0 (group-rank order)."""
    ax = symm.axis_for(group)
    C = _ext.load()
    t = t.contiguous()
    nbytes = t.numel() * t.element_size()
    if nbytes % 4:
        raise NotImplementedError("fused all-gather needs a multiple of 4 bytes per rank")
    out = torch.empty((ax.p * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if nbytes == 0:
        return out
    ax.ensure(nbytes)
    epoch, buf = ax.next_op()
    base = out.data_ptr()
    C.push_copy(t, ax.push_targets(buf) + [base + ax.rank * nbytes])
    remote, local = ax.sync(buf)
    C.gather_slots(ax.recv_slots(buf), [base + q * nbytes for q in ax.peers], nbytes, remote, local,
                   epoch, ax.timeout_ms, KID_GATHER, opc.status_buffer(t.device))
    opc._count(2)
    return out


def all_reduce_bf16(t: torch.Tensor, group) -> torch.Tensor:
    """In-place SUM all-reduce of a contiguous bf16 matrix whose width is a multiple of 8."""
    assert t.dtype == torch.bfloat16 and t.is_contiguous()
    t2 = t.view(-1, t.shape[-1]) if t.dim() > 1 else t.view(1, -1)
    if t2.numel() == 0:
        return t
    ax = symm.axis_for(group)
    if not _push_path(ax, t2.numel() * 2):
        dist.all_reduce(t, group=group)
        return t
    ax.ensure(t2.numel() * 2)
    epoch, buf = ax.next_op()
    _ext.load().push_copy(t2, ax.push_targets(buf))
    opc._count(1)
    _reduce(ax, t2, buf, epoch, False, None, KID_BARRIER)
    return t


def supports(t: torch.Tensor) -> bool:
    """Whether ``t`` can go through the peer-memory all-reduce."""
    if not t.is_cuda or not t.is_contiguous():
        return False
    if t.dtype == torch.float32:
        return True
    return t.dtype == torch.bfloat16 and t.dim() >= 1 and t.shape[-1] % 8 == 0
