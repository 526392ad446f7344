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


def relu_dropout(x, p: float = 0.0, seed: int = 0, index_offset: int = 0, training: bool = True):
    """``dropout(relu(x), p)`` with a reproducible, storage-free mask."""
    return ReluDropoutFunction.apply(x, p if training else 0.0, seed, index_offset)
