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
#   2 = tensor-core kernel (gathered rows staged in shared memory by cp.async, warp MMAs),
#   0 = the older warp-MMA accumulation inside the CUDA-core kernel's structure (kept for comparison).
SPMM_VARIANT = int(os.environ.get("PLEXUS_SPMM_VARIANT", "2"))
SPMM_MMA_STAGES = int(os.environ.get("PLEXUS_SPMM_MMA_STAGES", "0"))  # 0: chosen from the row size
# tensor-core kernel: rows longer than this are cut in pieces across warps; cost of a block of rows
SPMM_MMA_LONG_ROW = int(os.environ.get("PLEXUS_SPMM_MMA_LONG_ROW", "4096"))
SPMM_MMA_BLOCK_COST = int(os.environ.get("PLEXUS_SPMM_MMA_BLOCK_COST", "4096"))

# per-row constant added to the nonzero count when balancing row blocks, and the cost of a block
SPMM_ROW_COST = 8
SPMM_BLOCK_COST = 1024


class SpmmSchedule:
    """Device-side work schedule of one CSR matrix (or row range), built once and cached."""

    __slots__ = ("block_start", "piece_beg", "piece_end", "long_rows", "long_piece_start", "launches")


def spmm_schedule(crow: torch.Tensor, r0: int, r1: int, owner=None) -> SpmmSchedule:
    """Row blocks of about equal cost plus the pieces of rows longer than the kernel's piece size.

    The result is cached on ``owner`` (the sparse tensor object), so it lives exactly as long
    as the matrix it describes.
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
    key = (r0, r1)
    if cache is not None and key in cache:
        return cache[key]
    _schedules = cache if cache is not None else {}
    piece = _ext.load().spmm_piece_size()
    dev = crow.device
    i32 = dict(dtype=torch.int32, device=dev)
    sch = SpmmSchedule()
    rows = r1 - r0
    if rows <= 0:
        empty = torch.empty(0, **i32)
        sch.block_start = sch.piece_beg = sch.piece_end = sch.long_rows = sch.long_piece_start = empty
        sch.launches = 0
        _schedules[key] = sch
        return sch
    beg = crow[r0:r1].to(torch.int64)
    deg = crow[r0 + 1 : r1 + 1].to(torch.int64) - beg
    is_long = deg > piece
    cost = torch.where(is_long, torch.zeros_like(deg), deg) + SPMM_ROW_COST
    wcum = torch.cumsum(cost, 0)
    total = int(wcum[-1])
    nb = max(1, min(rows, total // SPMM_BLOCK_COST))
    targets = (torch.arange(1, nb, device=dev, dtype=torch.float64) * (total / nb)).to(torch.int64)
    inner = torch.searchsorted(wcum, targets, right=True)
    sch.block_start = (torch.cat([
        torch.zeros(1, dtype=torch.int64, device=dev), inner,
        torch.full((1,), rows, dtype=torch.int64, device=dev)]) + r0).to(torch.int32)
    idx = torch.nonzero(is_long).flatten()
    if idx.numel():
        ldeg, lbeg = deg[idx], beg[idx]
        npieces = (ldeg + piece - 1) // piece
        pstart = torch.zeros(idx.numel() + 1, dtype=torch.int64, device=dev)
        pstart[1:] = torch.cumsum(npieces, 0)
        owner = torch.repeat_interleave(torch.arange(idx.numel(), device=dev), npieces)
        k = torch.arange(int(pstart[-1]), device=dev) - pstart[:-1][owner]
        pb = lbeg[owner] + k * piece
        pe = torch.minimum(pb + piece, (lbeg + ldeg)[owner])
        sch.piece_beg, sch.piece_end = pb.to(torch.int32), pe.to(torch.int32)
        sch.long_rows = (idx + r0).to(torch.int32)
        sch.long_piece_start = pstart.to(torch.int32)
        sch.launches = 3
    else:
        empty = torch.empty(0, **i32)
        sch.piece_beg = sch.piece_end = sch.long_rows = sch.long_piece_start = empty
        sch.launches = 1
    _schedules[key] = sch
    return sch


class SpmmMmaSchedule:
    """Work items of the tensor-core SpMM for one matrix (or row range); see ``spmm_mma_schedule``."""

    __slots__ = ("items", "num_pieces", "long_piece_start", "long_counter")


def spmm_mma_schedule(crow: torch.Tensor, r0: int, r1: int, owner=None) -> SpmmMmaSchedule:
    """Work items of the tensor-core kernel for rows ``[r0, r1)``, built once per matrix on the device.

    * Rows longer than ``SPMM_MMA_LONG_ROW`` nonzeros are cut in equal pieces (multiples of 16
      nonzeros); a warp accumulates one piece into an fp32 partial row and the warp that delivers
      the last piece of a row sums the pieces in index order.
    * The other rows form blocks of consecutive rows of about ``SPMM_MMA_BLOCK_COST`` nonzeros
      (+ a per-row constant) each; a block never contains a long row, so its nonzeros are one
      contiguous range of the CSR arrays.

    ``items`` is int32 ``[n, 4]``: the pieces first (``row, -(long id + 1), first nnz, last nnz + 1``),
    then the blocks (``first row, last row + 1, 0, 0``).
    """
    cache = None
    if owner is not None:
        cache = getattr(owner, "_plx_spmm_mma_schedules", None)
        if cache is None:
            cache = {}
            try:
                owner._plx_spmm_mma_schedules = cache
            except Exception:
                cache = None
    key = (r0, r1, SPMM_MMA_BLOCK_COST, SPMM_MMA_LONG_ROW)
    if cache is not None and key in cache:
        return cache[key]
    dev = crow.device
    i32 = dict(dtype=torch.int32, device=dev)
    sch = SpmmMmaSchedule()
    rows = r1 - r0
    beg = crow[r0:r1].to(torch.int64)
    deg = crow[r0 + 1 : r1 + 1].to(torch.int64) - beg
    is_long = deg > SPMM_MMA_LONG_ROW
    # ---- pieces of the long rows
    lidx = torch.nonzero(is_long).flatten()
    if lidx.numel():
        ldeg, lbeg = deg[lidx], beg[lidx]
        want = (ldeg + SPMM_MMA_LONG_ROW - 1) // SPMM_MMA_LONG_ROW
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
        sch.long_counter = torch.zeros(lidx.numel(), **i32)
    else:
        pieces = torch.empty((0, 4), dtype=torch.int64, device=dev)
        sch.long_piece_start = torch.empty(0, **i32)
        sch.long_counter = torch.empty(0, **i32)
    sch.num_pieces = int(pieces.shape[0])
    # ---- blocks of the other rows: a new block where the accumulated cost crosses a multiple of the
    #      block cost, and after every long row
    sidx = torch.nonzero(~is_long).flatten()
    if sidx.numel():
        cost = deg[sidx] + SPMM_ROW_COST
        wcum = torch.cumsum(cost, 0)
        blk = (wcum - cost) // SPMM_MMA_BLOCK_COST
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
    """Whether :func:`spmm` can finish an all-reduce inside the kernel for these operands (the
    tensor-core kernel must be the one that runs, and one launch must cover all columns)."""
    if SPMM_VARIANT != 2 or H.dtype != torch.bfloat16 or H.shape[1] % 8 or H.shape[1] > 256:
        return False
    r0, r1 = row_range if row_range is not None else (0, A.shape[0])
    return r1 > r0


def spmm(A, H, relu_mask=None, row_range: Optional[Tuple[int, int]] = None, out_dtype=None, out=None,
         push_ptrs=(), push_ld=0, variant=None, push_seg=(0, 0), tile_reduce=None):
    """``push_ptrs``: this rank's receive slots in the peers' workspaces (fused collective).
    ``push_seg = (rows per owner, this rank's position)``: reduce-scatter push (each row goes only
    to the rank that owns it) instead of the broadcast push.
    ``variant``: see ``SPMM_VARIANT`` (default: the tensor-core kernel for bf16 features).
    ``tile_reduce = (slots, remote_sig, local_sig, me, timeout_ms, tile_rows, local_done_ptr)``:
    finish the all-reduce over the push peers inside the kernel (the mask is applied after the
    sum); only with the tensor-core kernel, see :func:`spmm_supports_tile_reduce`."""
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
    if variant == 2 and H.dtype == torch.bfloat16 and H.shape[1] % 8 == 0 and r1 > r0:
        sch = spmm_mma_schedule(crow, r0, r1, owner=A)
        if sch.num_pieces == 0 or H.shape[1] <= 256:
            tr = tile_reduce if tile_reduce is not None else ([], [], [], 0, 0.0, 0, 0)
            scratch = (_scratch_floats(sch.num_pieces * H.shape[1], H.device) if sch.num_pieces
                       else _EMPTY_F32(H.device))
            C.spmm_mma(crow, col, val, H, out, relu_mask, r0, sch.items, sch.num_pieces, sch.long_piece_start,
                       sch.long_counter, scratch, list(push_ptrs), int(push_ld),
                       SPMM_MMA_STAGES, int(push_seg[0]), int(push_seg[1]), status_buffer(H.device),
                       list(tr[0]), list(tr[1]), list(tr[2]), int(tr[3]), float(tr[4]), int(tr[5]), int(tr[6]))
            _count(-(-H.shape[1] // 256))
            if out_dtype is not None and out_dtype != out.dtype:
                out = out.to(out_dtype)
            return out
    if tile_reduce is not None:
        raise RuntimeError("spmm: the in-kernel all-reduce needs the tensor-core kernel")
    if variant == 2:
        variant = 1
    sch = spmm_schedule(crow, r0, r1, owner=A)
    npieces = sch.piece_beg.numel()
    scratch = _scratch_floats(npieces * C.spmm_scratch_per_piece(H), H.device) if npieces else _EMPTY_F32(H.device)
    C.spmm_csr(crow, col, val, H, out, relu_mask, r0, sch.block_start, sch.piece_beg, sch.piece_end,
               sch.long_rows, sch.long_piece_start, scratch, list(push_ptrs), int(push_ld),
               variant, int(push_seg[0]), int(push_seg[1]))
    _count(sch.launches)
    if out_dtype is not None and out_dtype != out.dtype:
        out = out.to(out_dtype)
    return out


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
    ``tile_reduce = (slots, remote_sig, local_sig, base, me, timeout_ms)``: finish the all-reduce
    over the push peers inside the kernel (ReLU / mask applied after the sum)."""
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
    tr = tile_reduce if tile_reduce is not None else ([], [], [], 0, 0, 0.0)
    C.gemm_nt(a, bt, out, bool(relu), st, max_stages, ctas, nb, list(push_ptrs), int(push_ld), relu_mask,
              int(push_seg[0]), int(push_seg[1]), list(tr[0]), list(tr[1]), list(tr[2]), int(tr[3]), int(tr[4]),
              float(tr[5]))
    _count(1)
    return out


def relu_backward(grad, out):
    res = torch.empty_like(out)
    _ext.load().relu_bwd(grad.contiguous(), out.contiguous(), res)
    _count(1)
    return res


def xent_local_stats(logits, class_offset, num_classes):
    R = logits.shape[0]
    rmax = torch.empty(R, dtype=torch.float32, device=logits.device)
    rsum = torch.empty(R, dtype=torch.float32, device=logits.device)
    _ext.load().xent_stats(logits, int(class_offset), int(num_classes), rmax, rsum)
    _count(1)
    return rmax, rsum


def xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, weight=None):
    loss = torch.zeros(1, dtype=torch.float32, device=logits.device)
    _ext.load().xent_loss(logits, target, gmax, gsum, weight, int(row_offset), int(class_offset),
                          int(num_nodes), loss)
    _count(1)
    return loss.reshape(())


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
