"""ReLU followed by inverted dropout, as one op (stand-alone version for unfused paths).

The keep mask is a pure function of ``(seed, element index)`` (the counter-based hash of
``data/synthetic.py``), so forward and backward agree without storing a mask, a rank can apply
the op to its shard with ``index_offset`` = position of the shard in the full tensor, and the
CPU and CUDA versions drop the same elements.  The reference has no dropout; the op exists for
models that want it between GCN layers.
"""

from __future__ import annotations

import torch

from ..data.synthetic import _lsr, hash_stream


def keep_mask(numel: int, p: float, seed: int, index_offset: int = 0, device="cpu") -> torch.Tensor:
    idx = torch.arange(index_offset, index_offset + numel, dtype=torch.int64, device=device)
    return _lsr(hash_stream(seed, 7000, idx), 32) >= int(p * 4294967296.0)


class ReluDropoutFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, index_offset):
        ctx.p, ctx.seed, ctx.offset = float(p), int(seed), int(index_offset)
        xc = x.contiguous()
        if xc.is_cuda:
            from . import _ext, cuda as opc

            y = _ext.load().relu_dropout(xc, None, ctx.p, ctx.seed, ctx.offset)
            opc._count(1)
        else:
            y = torch.relu(xc)
            if ctx.p > 0:
                keep = keep_mask(xc.numel(), ctx.p, ctx.seed, ctx.offset).view_as(xc)
                y = (y.float() * keep / (1.0 - ctx.p)).to(x.dtype)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad):
        (y,) = ctx.saved_tensors
        g = grad.contiguous()
        if g.is_cuda:
            from . import _ext, cuda as opc

            out = _ext.load().relu_dropout(y, g, ctx.p, ctx.seed, ctx.offset)
            opc._count(1)
        else:
            out = (g.float() * (y > 0) / (1.0 - ctx.p)).to(g.dtype)
        return out, None, None, None


def keep_mask_2d(rows: int, cols: int, p: float, seed: int, row0: int, col0: int, full_cols: int,
                 device="cpu", chunk_rows: int = 1 << 20) -> torch.Tensor:
    """Keep mask of the block ``[row0, row0+rows) x [col0, col0+cols)`` of a matrix with ``full_cols``
    columns: element ``(r, c)`` is hashed by its global position ``r * full_cols + c``, so every
    sharding of the matrix (and every replica of a shard) drops the same elements."""
    out = torch.empty((rows, cols), dtype=torch.bool, device=device)
    c = torch.arange(col0, col0 + cols, dtype=torch.int64, device=device)
    thr = int(p * 4294967296.0)
    for a in range(0, rows, chunk_rows):
        b = min(rows, a + chunk_rows)
        r = torch.arange(row0 + a, row0 + b, dtype=torch.int64, device=device)
        idx = r[:, None] * full_cols + c[None, :]
        out[a:b] = _lsr(hash_stream(seed, 7000, idx), 32) >= thr
    return out


class ReluDropout2dFunction(torch.autograd.Function):
    """``dropout(relu(x))`` on a 2-D shard with the position-keyed mask of :func:`keep_mask_2d`."""

    @staticmethod
    def forward(ctx, x, p, seed, row0, col0, full_cols):
        ctx.p = float(p)
        y = torch.relu(x)
        if ctx.p > 0:
            keep = keep_mask_2d(x.shape[0], x.shape[1], ctx.p, int(seed), int(row0), int(col0), int(full_cols),
                                device=x.device)
            y = (y * keep).mul_(1.0 / (1.0 - ctx.p)) if y.dtype != torch.bfloat16 else (
                (y.float() * keep) * (1.0 / (1.0 - ctx.p))).to(x.dtype)
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad):
        (y,) = ctx.saved_tensors
        out = (grad.float() * (y > 0) * (1.0 / (1.0 - ctx.p))).to(grad.dtype) if grad.dtype == torch.bfloat16 \
            else grad * (y > 0) * (1.0 / (1.0 - ctx.p))
        return out, None, None, None, None, None


def relu_dropout_2d(x, p: float, seed: int, row0: int, col0: int, full_cols: int, training: bool = True):
    """Sharding-invariant ``dropout(relu(x), p)`` for a block of a row/column-sharded activation."""
    return ReluDropout2dFunction.apply(x, p if training else 0.0, seed, row0, col0, full_cols)


def relu_dropout(x, p: float = 0.0, seed: int = 0, index_offset: int = 0, training: bool = True):
    """``dropout(relu(x), p)`` with a reproducible, storage-free mask."""
    return ReluDropoutFunction.apply(x, p if training else 0.0, seed, index_offset)
