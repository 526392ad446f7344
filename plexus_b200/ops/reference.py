"""Plain PyTorch versions of every op (CPU path and numerical oracle).

These run wherever torch runs.  They define the semantics the sm_100a kernels
in ``plexus_b200/csrc`` are tested against; on a CUDA device the dispatcher in
``plexus_b200.ops`` never routes here.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch


def _acc(t: torch.Tensor) -> torch.Tensor:
    """Accumulation copy: fp32 for 16/32-bit inputs, fp64 stays fp64."""
    return t if t.dtype == torch.float64 else t.float()


def extract_csr_submatrix(csr_matrix: torch.Tensor, start_row: int, end_row: int) -> torch.Tensor:
    """Rows ``[start_row, end_row)`` of a CSR matrix as a new CSR matrix.

    Reference: plexus/gcn_conv.py:25-64.
    """
    crow, col, val = csr_matrix.crow_indices(), csr_matrix.col_indices(), csr_matrix.values()
    lo, hi = int(crow[start_row]), int(crow[end_row])
    sub_crow = crow[start_row : end_row + 1] - crow[start_row]
    return torch.sparse_csr_tensor(
        sub_crow, col[lo:hi], val[lo:hi], size=(end_row - start_row, csr_matrix.shape[1]),
        check_invariants=False,
    )


def spmm(A: torch.Tensor, H: torch.Tensor, relu_mask: Optional[torch.Tensor] = None,
         row_range: Optional[Tuple[int, int]] = None, out_dtype=None) -> torch.Tensor:
    """``A @ H`` with fp32 accumulation; optional ``* (relu_mask > 0)`` epilogue."""
    if row_range is not None:
        A = extract_csr_submatrix(A, row_range[0], row_range[1])
    Hf = _acc(H)
    vals = A.values()
    if vals.dtype != Hf.dtype:
        A = torch.sparse_csr_tensor(A.crow_indices(), A.col_indices(), vals.to(Hf.dtype), size=A.shape,
                                    check_invariants=False)
    out = torch.sparse.mm(A, Hf)
    if relu_mask is not None:
        out = out * (relu_mask > 0).to(out.dtype)
    return out.to(out_dtype or H.dtype)


def gemm(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False,
         relu: bool = False, out_dtype=None) -> torch.Tensor:
    """``op(a) @ op(b)`` with fp32 accumulation and optional ReLU."""
    x = _acc(a).t() if trans_a else _acc(a)
    y = _acc(b).t() if trans_b else _acc(b)
    if x.dtype != y.dtype:
        x, y = x.to(torch.promote_types(x.dtype, y.dtype)), y.to(torch.promote_types(x.dtype, y.dtype))
    out = x @ y
    if relu:
        out = torch.relu(out)
    return out.to(out_dtype or a.dtype)


def relu_backward(grad: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    return grad * (out > 0).to(grad.dtype)


def xent_local_stats(logits: torch.Tensor, class_offset: int, num_classes: int):
    """Per-row (max, sum exp(l - max)) over this rank's valid classes (fp32)."""
    C = logits.shape[1]
    valid = (torch.arange(C, device=logits.device) + class_offset) < num_classes
    lf = _acc(logits).masked_fill(~valid.unsqueeze(0), float("-inf"))
    m = lf.max(dim=1).values if C > 0 else torch.full((logits.shape[0],), float("-inf"), dtype=lf.dtype)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    s = torch.exp(lf - m_safe.unsqueeze(1)).sum(dim=1)
    return m, s


def xent_stats(logits, class_offset, num_classes, target=None, row_offset=0, num_nodes=0, weight=None):
    """``[2, R]`` statistics and, with ``target`` (classes not sharded), the loss."""
    m, s = xent_local_stats(logits, class_offset, num_classes)
    loss = None
    if target is not None:
        loss = xent_combine_loss(logits, target, m, s, row_offset, class_offset, num_nodes, weight)
    return torch.stack([m, s]), loss


def xent_combine(logits, target, pairs, row_offset, class_offset, num_nodes, weight=None):
    """Combine every class shard's (max, sum exp) in rank order; loss terms of the local targets."""
    lmax, lsum = pairs[:, 0], pairs[:, 1]
    gmax = lmax.max(dim=0).values
    # a shard holding only padded classes reports (-inf, 0)
    finite = torch.where(torch.isinf(lmax), torch.full_like(lmax, -1e30), lmax)
    gsum = (lsum * torch.exp(finite - gmax)).sum(dim=0)
    loss = xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, weight)
    return torch.stack([gmax, gsum]), loss


def xent_combine_loss(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, weight=None):
    """Sum over local rows of ``-log softmax[target]`` restricted to local classes.

    ``gmax`` / ``gsum`` are the row statistics reduced over the class axis.
    Rows beyond ``num_nodes`` and rows with a negative label contribute 0.
    """
    R, C = logits.shape
    rows = torch.arange(R, device=logits.device) + row_offset
    valid_row = (rows < num_nodes) & (target >= 0)
    local = target - class_offset
    has = valid_row & (local >= 0) & (local < C)
    idx = local.clamp(0, max(C - 1, 0))
    picked = _acc(logits).gather(1, idx.unsqueeze(1)).squeeze(1) if C > 0 else torch.zeros(R, dtype=gmax.dtype)
    logp = picked - gmax - torch.log(gsum)
    contrib = torch.where(has, -logp, torch.zeros_like(logp))
    if weight is not None:
        contrib = contrib * weight
    return contrib.sum()


def xent_grad(logits, target, gmax, gsum, row_offset, class_offset, num_nodes, num_classes,
              scale, out_dtype=None):
    """``(softmax - onehot) * scale`` on valid rows, 0 elsewhere and on padded classes."""
    R, C = logits.shape
    rows = torch.arange(R, device=logits.device) + row_offset
    valid_row = (rows < num_nodes) & (target >= 0)
    cls = torch.arange(C, device=logits.device) + class_offset
    valid_cls = cls < num_classes
    p = torch.exp(_acc(logits) - gmax.unsqueeze(1)) / gsum.unsqueeze(1)
    p = p * valid_cls.unsqueeze(0)
    onehot = (cls.unsqueeze(0) == target.unsqueeze(1)).to(p.dtype)
    g = (p - onehot) * valid_row.unsqueeze(1) * scale
    return g.to(out_dtype or logits.dtype)


def adam_step(params, grads, exp_avgs, exp_avg_sqs, masters, step, lr, beta1, beta2, eps,
              weight_decay, decoupled=True):
    """AdamW (``decoupled``) or Adam-with-L2 update, fp32 math on the master copy."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    for p, g, m, v, w in zip(params, grads, exp_avgs, exp_avg_sqs, masters):
        wf = w if w is not None else p
        gf = _acc(g)
        if weight_decay != 0.0:
            if decoupled:
                wf.mul_(1.0 - lr * weight_decay)
            else:
                gf = gf + weight_decay * wf
        m.mul_(beta1).add_(gf, alpha=1.0 - beta1)
        v.mul_(beta2).addcmul_(gf, gf, value=1.0 - beta2)
        denom = (v / bc2).sqrt_().add_(eps)
        wf.addcdiv_(m, denom, value=-lr / bc1)
        if w is not None:
            p.copy_(w)
