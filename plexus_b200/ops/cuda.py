"""CUDA implementations of the ops: thin wrappers over the kernels in ``_C``.

Storage dtype on the device is bf16 (features, activations, their gradients)
with fp32 accumulation; weights and optimizer state stay fp32.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import os

import torch

from . import _ext

# (max_stages, ctas_limit, column-block width) launch shapes of the tcgen05 GEMM tried by the tuner;
# 0 = default
GEMM_VARIANTS = [(0, 0, 0), (0, 0, 256), (0, 0, 128), (0, 0, 64), (4, 0, 0), (0, 74, 0)]

# number of kernels of this package launched so far (counted where they are launched)
launch_count = 0


def _count(n: int) -> None:
    global launch_count
    launch_count += n


_status: Dict[int, torch.Tensor] = {}
_scratch: Dict[int, torch.Tensor] = {}


def status_buffer(device=None) -> torch.Tensor:
    """int32[8] status words written by kernels whose bounded waits gave up."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx not in _status:
        _status[idx] = torch.zeros(8, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device=None) -> None:
    """Raise if any kernel recorded a timeout since the last check (synchronises)."""
    from ..parallel.watchdog import raise_on_device_status

    raise_on_device_status(status_buffer(device))


def _scratch_floats(n: int, device) -> torch.Tensor:
    idx = device.index
    buf = _scratch.get(idx)
    if buf is None or buf.numel() < n:
        buf = torch.empty(max(n, 1 << 20), dtype=torch.float32, device=device)
        _scratch[idx] = buf
    return buf


def _csr_parts(A):
    crow, col, val = A.crow_indices(), A.col_indices(), A.values()
    if crow.dtype != torch.int32 or col.dtype != torch.int32:
        raise TypeError("CUDA SpMM needs int32 CSR indices (build shards with plexus_b200's loader)")
    if val.dtype != torch.float32:
        val = val.float()
    return crow, col, val


# SpMM kernel variants:
#   1 = CUDA-core kernel (packed fp32x2 multiply-adds; also the only one for fp32 features),
#   2 = tensor-core kernel (gathered rows staged in shared memory by cp.async, warp MMAs; bf16 only).
# Measured on B200 the CUDA-core kernel is the faster one at every width of the GCN configurations
# (e.g. 1.07 ms against 1.33 ms on a 1.2M x 1.2M shard with 31M nonzeros at 128 columns), so it is
# the default; the tensor-core kernel stays selectable.
SPMM_VARIANT = int(os.environ.get("PLEXUS_SPMM_VARIANT", "1"))
SPMM_MMA_STAGES = int(os.environ.get("PLEXUS_SPMM_MMA_STAGES", "0"))  # 0: chosen from the row size
# per-row constant added to the nonzero count when balancing row blocks
SPMM_ROW_COST = 8
# (rows longer than this are cut in pieces across warps, cost of a block of rows) per variant
SPMM_LONG_ROW = {1: int(os.environ.get("PLEXUS_SPMM_LONG_ROW", "1024")),
                 2: int(os.environ.get("PLEXUS_SPMM_MMA_LONG_ROW", "4096"))}
SPMM_BLOCK_COST = {1: int(os.environ.get("PLEXUS_SPMM_BLOCK_COST", "1024")),
                   2: int(os.environ.get("PLEXUS_SPMM_MMA_BLOCK_COST", "4096"))}


class SpmmSchedule:
    """Work items of an SpMM kernel for one matrix (or row range); see ``spmm_schedule``."""

    __slots__ = ("items", "num_pieces", "long_piece_start", "long_counter")


def spmm_schedule(crow: torch.Tensor, r0: int, r1: int, owner=None, variant: int = 1) -> SpmmSchedule:
    """Work items of an SpMM kernel for rows ``[r0, r1)``, built once per matrix on the device.

    * Rows longer than ``SPMM_LONG_ROW[variant]`` nonzeros are cut in equal pieces (multiples of 16
      nonzeros); a warp accumulates one piece into an fp32 partial row and the warp that delivers
      the last piece of a row sums the pieces in index order.
    * The other rows form blocks of consecutive rows of about ``SPMM_BLOCK_COST[variant]`` nonzeros
      (+ a per-row constant) each; a block never contains a long row, so its nonzeros are one
      contiguous range of the CSR arrays.

    ``items`` is int32 ``[n, 4]``: the pieces first (``row, -(long id + 1), first nnz, last nnz + 1``),
    then the blocks (``first row, last row + 1, 0, 0``).
    """
    cache = None
    if owner is not None:
        cache = getattr(owner, "_plx_spmm_schedules", None)
        if cache is None:
            cache = {}
            try:
                owner._plx_spmm_schedules = cache
            except Exception:
                cache = None
    long_row, block_cost = SPMM_LONG_ROW[variant], SPMM_BLOCK_COST[variant]
    key = (r0, r1, block_cost, long_row)
    if cache is not None and key in cache:
        return cache[key]
    dev = crow.device
    i32 = dict(dtype=torch.int32, device=dev)
    sch = SpmmSchedule()
    rows = r1 - r0
    beg = crow[r0:r1].to(torch.int64)
    deg = crow[r0 + 1 : r1 + 1].to(torch.int64) - beg
    is_long = deg > long_row
    # ---- pieces of the long rows
    lidx = torch.nonzero(is_long).flatten()
    if lidx.numel():
        ldeg, lbeg = deg[lidx], beg[lidx]
        want = (ldeg + long_row - 1) // long_row
        plen = ((ldeg + want - 1) // want + 15) // 16 * 16
        npieces = (ldeg + plen - 1) // plen
        pstart = torch.zeros(lidx.numel() + 1, dtype=torch.int64, device=dev)
        pstart[1:] = torch.cumsum(npieces, 0)
        owner_of = torch.repeat_interleave(torch.arange(lidx.numel(), device=dev), npieces)
        k = torch.arange(int(pstart[-1]), device=dev) - pstart[:-1][owner_of]
        pb = lbeg[owner_of] + k * plen[owner_of]
        pe = torch.minimum(pb + plen[owner_of], (lbeg + ldeg)[owner_of])
        pieces = torch.stack([lidx[owner_of] + r0, -(owner_of + 1), pb, pe], dim=1)
        sch.long_piece_start = pstart.to(torch.int32)
        sch.long_counter = torch.zeros(lidx.numel() + 2, **i32)  # + the two work hand-out counters
    else:
        pieces = torch.empty((0, 4), dtype=torch.int64, device=dev)
        sch.long_piece_start = torch.empty(0, **i32)
        sch.long_counter = torch.zeros(2, **i32)
    sch.num_pieces = int(pieces.shape[0])
    # ---- blocks of the other rows: a new block where the accumulated cost crosses a multiple of the
    #      block cost, and after every long row
    sidx = torch.nonzero(~is_long).flatten()
    if sidx.numel():
        cost = deg[sidx] + SPMM_ROW_COST
        wcum = torch.cumsum(cost, 0)
        blk = (wcum - cost) // block_cost
        run = torch.cumsum(is_long.to(torch.int64), 0)[sidx]
        keyv = run * (int(blk[-1]) + 2) + blk
        first = torch.ones(sidx.numel(), dtype=torch.bool, device=dev)
        first[1:] = keyv[1:] != keyv[:-1]
        starts = torch.nonzero(first).flatten()
        ends = torch.cat([starts[1:], torch.full((1,), sidx.numel(), dtype=torch.int64, device=dev)])
        rb = sidx[starts] + r0
        re = sidx[ends - 1] + 1 + r0
        zeros = torch.zeros_like(rb)
        blocks = torch.stack([rb, re, zeros, zeros], dim=1)
    else:
        blocks = torch.empty((0, 4), dtype=torch.int64, device=dev)
    sch.items = torch.cat([pieces, blocks]).to(torch.int32).contiguous()
    if cache is not None:
        cache[key] = sch
    return sch


DEBUG = os.environ.get("PLEXUS_DEBUG", "0") not in ("", "0")


def validate_csr(A) -> None:
    """Check the structure of a sparse CSR shard on the device (row pointers start at 0, are
    monotone and end at nnz; every column index is inside the matrix).  Raises ``RuntimeError``
    naming the first violation.  Runs automatically once per matrix when ``PLEXUS_DEBUG=1``."""
    crow, col, _ = _csr_parts(A)
    st = status_buffer(col.device)
    _ext.load().csr_validate(crow, col, A.shape[0], A.shape[1], st)
    _count(1)
    check_status(col.device)


def spmm_supports_tile_reduce(A, H, row_range=None) -> bool:
    """Whether :func:`spmm` can finish an all-reduce inside the kernel for these operands."""
    if H.dtype != torch.bfloat16 or H.shape[1] % 8:
        return False
    if SPMM_VARIANT == 2 and H.shape[1] > 256:
        return False
    r0, r1 = row_range if row_range is not None else (0, A.shape[0])
    return r1 > r0


def spmm(A, H, relu_mask=None, row_range: Optional[Tuple[int, int]] = None, out_dtype=None, out=None,
         push_ptrs=(), push_ld=0, variant=None, push_seg=(0, 0), tile_reduce=None):
    """``push_ptrs``: this rank's receive slots in the peers' workspaces (fused collective).
    ``push_seg = (rows per owner, this rank's position)``: reduce-scatter push (each row goes only
    to the rank that owns it) instead of the broadcast push.
    ``variant``: see ``SPMM_VARIANT``.
    ``tile_reduce = (sentinel slots, me, timeout_ms)`` (``AxisComm.tile_reduce``): finish the
    all-reduce over the push peers inside the kernel (the mask is applied after the sum); the push
    must then go to the peers' sentinel slots.  See :func:`spmm_supports_tile_reduce`."""
    C = _ext.load()
    crow, col, val = _csr_parts(A)
    r0, r1 = row_range if row_range is not None else (0, A.shape[0])
    if H.shape[0] < A.shape[1]:
        raise ValueError(f"spmm: dense operand has {H.shape[0]} rows, the sparse one {A.shape[1]} columns")
    if not 0 <= r0 <= r1 <= A.shape[0]:
        raise ValueError(f"spmm: row range {(r0, r1)} outside the matrix")
    if DEBUG and not getattr(A, "_plx_validated", False):
        validate_csr(A)
        try:
            A._plx_validated = True
        except AttributeError:
            pass
    if H.stride(-1) != 1:
        H = H.contiguous()
    if out is None:
        out = torch.empty((r1 - r0, H.shape[1]), dtype=H.dtype, device=H.device)
    if relu_mask is not None and relu_mask.dtype != H.dtype:
        relu_mask = relu_mask.to(H.dtype)
    variant = SPMM_VARIANT if variant is None else int(variant)
    if variant not in (1, 2):
        raise ValueError("spmm: variant must be 1 (CUDA cores) or 2 (tensor cores)")
    if variant == 2 and not (H.dtype == torch.bfloat16 and H.shape[1] % 8 == 0):
        variant = 1
    if r1 == r0 or H.shape[1] == 0:
        return out if out_dtype in (None, out.dtype) else out.to(out_dtype)
    sch = spmm_schedule(crow, r0, r1, owner=A, variant=variant)
    if variant == 2 and sch.num_pieces and H.shape[1] > 256:
        variant = 1  # the tensor-core kernel sums pieces of at most 256 columns
        sch = spmm_schedule(crow, r0, r1, owner=A, variant=variant)
    per_piece = H.shape[1] if variant == 2 else C.spmm_scratch_per_piece(H)
    scratch = _scratch_floats(sch.num_pieces * per_piece, H.device) if sch.num_pieces else _EMPTY_F32(H.device)
    tr = tile_reduce if tile_reduce is not None else ([], 0, 0.0)
    C.spmm_items(variant == 2, crow, col, val, H, out, relu_mask, r0, sch.items, sch.num_pieces,
                 sch.long_piece_start, sch.long_counter, scratch, list(push_ptrs), int(push_ld), SPMM_MMA_STAGES,
                 int(push_seg[0]), int(push_seg[1]), status_buffer(H.device), list(tr[0]), int(tr[1]),
                 float(tr[2]), _push_limit(push_ptrs, out))
    if variant == 2:
        _count(-(-H.shape[1] // 256))
    else:
        # the items kernel, plus the launch that sums the pieces of the long rows (the fused
        # in-kernel form does that inside the one launch)
        _count(2 if sch.num_pieces and not len(tr[0]) else 1)
    if out_dtype is not None and out_dtype != out.dtype:
        out = out.to(out_dtype)
    return out


def _push_limit(push_ptrs, out) -> int:
    """Capacity of the receive slots in elements of ``out`` when the push targets carry one (a debug
    run, see ``parallel.symm.PushList``): the kernels then check every fused-collective store."""
    nbytes = getattr(push_ptrs, "limit_bytes", 0)
    return int(nbytes) // out.element_size() if nbytes else 0


def _EMPTY_F32(device):
    return torch.empty(0, dtype=torch.float32, device=device)


def _bf16(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.bfloat16:
        return t
    raise TypeError(
        "the CUDA GEMM path takes bf16 activations (fp32 accumulate); got "
        f"{t.dtype}. Initialise with dtype=torch.bfloat16."
    )


def gemm(a, b, trans_a=False, trans_b=False, relu=False, out_dtype=None, variant: int = 0,
         push_ptrs=(), push_ld=0, relu_mask=None, push_seg=(0, 0), out=None, tile_reduce=None):
    """``relu_mask`` (shape of the result): zero the result where the mask is not positive.
    ``push_ptrs`` / ``push_seg``: fused-collective epilogue, see :func:`spmm`.
    ``out``: optional destination of ``op(a) @ op(b)`` for the non-transposed-``a`` forms (rows
    contiguous, e.g. a row block of a larger matrix).
    ``tile_reduce = (sentinel slots, me, timeout_ms)`` (``AxisComm.tile_reduce``): finish the
    all-reduce over the push peers inside the kernel (ReLU / mask applied after the sum)."""
    C = _ext.load()
    st = status_buffer(a.device)
    max_stages, ctas, nb = GEMM_VARIANTS[variant]
    if trans_a and not trans_b:
        # out[Mw, Nw] = a[R, Mw]^T . b[R, Nw]   (fp32 result)
        a, b = _bf16(a), _bf16(b)
        if a.stride(-1) != 1:
            a = a.contiguous()
        if b.stride(-1) != 1:
            b = b.contiguous()
        Mw, Nw = a.shape[1], b.shape[1]
        out = torch.empty((Mw, Nw), dtype=torch.float32, device=a.device)
        parts = C.gemm_tn_parts(a.shape[0])
        C.gemm_tn(a, b, out, _scratch_floats(parts * Mw * Nw, a.device), st)
        _count(2)
        if relu:
            out = torch.relu_(out)
        return out if out_dtype in (None, torch.float32) else out.to(out_dtype)
    if trans_a:
        raise NotImplementedError("gemm with both operands transposed is not used by the layers")
    a = _bf16(a)
    if a.stride(-1) != 1:
        a = a.contiguous()
    if trans_b:
        bt = b if b.dtype == torch.bfloat16 else b.to(torch.bfloat16)  # [N, K], K contiguous
        if not bt.is_contiguous():
            bt = bt.contiguous()
    else:
        # b is [K, N]: the tensor cores want it K-major, i.e. b^T [N, K]
        bt = torch.empty((b.shape[1], b.shape[0]), dtype=torch.bfloat16, device=b.device)
        C.prep_weight(b.contiguous(), None, bt)
        _count(1)
    if out is None:
        out = torch.empty((a.shape[0], bt.shape[0]), dtype=out_dtype or a.dtype, device=a.device)
    elif tuple(out.shape) != (a.shape[0], bt.shape[0]) or out.stride(-1) != 1:
        raise ValueError("gemm: out has the wrong shape or layout")
    if relu_mask is not None and relu_mask.dtype != out.dtype:
        relu_mask = relu_mask.to(out.dtype)
    tr = tile_reduce if tile_reduce is not None else ([], 0, 0.0)
    C.gemm_nt(a, bt, out, bool(relu), st, max_stages, ctas, nb, list(push_ptrs), int(push_ld), relu_mask,
              int(push_seg[0]), int(push_seg[1]), list(tr[0]), int(tr[1]), float(tr[2]), _push_limit(push_ptrs, out))
    _count(1)
    return out


def relu_backward(grad, out):
    res = torch.empty_like(out)
    _ext.load().relu_bwd(grad.contiguous(), out.contiguous(), res)
    _count(1)
    return res


def xent_stats(logits, class_offset, num_classes, target=None, row_offset=0, num_nodes=0, weight=None,
               push_ptrs=()):
    """fp32 ``[2, R]`` per-row (max, sum exp) over this rank's classes.  With ``target`` (classes not
    sharded) the same launch adds up the loss: returns ``(stats, loss)``, else ``(stats, None)``.
    ``push_ptrs``: this rank's receive slots (``[2, R]`` floats) on the peers of the class axis; the
    kernel stores every pair there as well."""
    R = logits.shape[0]
    stats = torch.empty((2, R), dtype=torch.float32, device=logits.device)
    loss = None if target is None else torch.zeros(1, dtype=torch.float32, device=logits.device)
    _ext.load().xent_stats(logits, int(class_offset), int(num_classes), stats, target, weight, int(row_offset),
                           int(num_nodes), loss, list(push_ptrs))
    _count(1)
    return stats, (None if loss is None else loss.reshape(()))


def xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, weight=None):
    """``pairs`` fp32 ``[P, 2, R]`` (every class shard's statistics) -> ``(stats [2, R], loss)``."""
    pairs = pairs.contiguous()
    R = logits.shape[0]
    ptrs = [pairs.data_ptr() + q * 2 * R * 4 for q in range(pairs.shape[0])]
    return xent_combine_ptrs(logits, target, ptrs, row_offset, class_offset, num_nodes, weight, _keep=pairs)


def xent_combine_ptrs(logits, target, pair_ptrs, row_offset, class_offset, num_nodes, weight=None, sync=None,
                      like=None, _keep=None):
    """Like :func:`xent_combine` with the statistics given by device address (rank order).
    ``sync = (remote flags, local flags, epoch, timeout_ms)``: the kernel starts with that flag
    barrier (the pairs were pushed into this rank's receive slots)."""
    R = logits.shape[0]
    stats = torch.empty((2, R), dtype=torch.float32, device=logits.device)
    loss = torch.zeros(1, dtype=torch.float32, device=logits.device)
    remote, local, epoch, timeout_ms = sync if sync is not None else ([], [], 0, 0.0)
    _ext.load().xent_combine(logits, target, [int(p) for p in pair_ptrs], weight, int(row_offset), int(class_offset),
                             int(num_nodes), stats, loss, list(remote), list(local), int(epoch), float(timeout_ms),
                             status_buffer(logits.device))
    _count(1)
    return stats, loss.reshape(())


def xent_local_stats(logits, class_offset, num_classes):
    stats, _ = xent_stats(logits, class_offset, num_classes)
    return stats[0], stats[1]


def xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, weight=None):
    pairs = torch.stack([gmax.float(), gsum.float()]).unsqueeze(0)
    return xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, weight)[1]


def xent_grad(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, num_classes, scale,
              out_dtype=None):
    if not torch.is_tensor(scale):
        scale = torch.tensor([float(scale)], dtype=torch.float32, device=logits.device)
    scale = scale.to(torch.float32).reshape(1)
    grad = torch.empty_like(logits)
    _ext.load().xent_grad(logits, target, gmax, gsum, scale, int(row_offset), int(class_offset),
                          int(num_nodes), int(num_classes), grad)
    _count(1)
    return grad if out_dtype in (None, grad.dtype) else grad.to(out_dtype)


def adam_step(params, grads, exp_avgs, exp_avg_sqs, masters, step, lr, beta1, beta2, eps,
              weight_decay, decoupled=True):
    _ext.load().adam_multi(list(params), list(grads), list(exp_avgs), list(exp_avg_sqs), list(masters),
                           int(step), float(lr), float(beta1), float(beta2), float(eps),
                           float(weight_decay), bool(decoupled))
    _count((len(params) + 23) // 24)
