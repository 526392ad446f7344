"""CUDA implementations of the ops: thin wrappers over the kernels in ``_C``.

Storage dtype on the device is bf16 (features, activations, their gradients)
with fp32 accumulation; weights and optimizer state stay fp32.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import _ext

# (max_stages, ctas_limit) launch shapes of the tcgen05 GEMM tried by the tuner; 0 = default
GEMM_VARIANTS = [(0, 0), (4, 0), (3, 0), (2, 0), (0, 74), (0, 296)]

# number of kernels of this package launched so far (counted where they are launched)
launch_count = 0


def _count(n: int) -> None:
    global launch_count
    launch_count += n


_status: Dict[int, torch.Tensor] = {}
_scratch: Dict[int, torch.Tensor] = {}
_long_rows: Dict[Tuple[int, int], torch.Tensor] = {}


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


def long_rows_of(crow: torch.Tensor) -> torch.Tensor:
    """Rows with more nonzeros than the kernel's long-row threshold (cached per matrix)."""
    key = (crow.data_ptr(), crow.numel())
    got = _long_rows.get(key)
    if got is None:
        thr = _ext.load().spmm_long_row_threshold()
        deg = crow[1:] - crow[:-1]
        got = torch.nonzero(deg > thr).flatten().to(torch.int32)
        _long_rows[key] = got
    return got


def spmm(A, H, relu_mask=None, row_range: Optional[Tuple[int, int]] = None, out_dtype=None, out=None):
    C = _ext.load()
    crow, col, val = _csr_parts(A)
    r0, r1 = row_range if row_range is not None else (0, A.shape[0])
    if H.stride(-1) != 1:
        H = H.contiguous()
    if out is None:
        out = torch.empty((r1 - r0, H.shape[1]), dtype=H.dtype, device=H.device)
    if relu_mask is not None and relu_mask.dtype != H.dtype:
        relu_mask = relu_mask.to(H.dtype)
    lr = long_rows_of(crow)
    C.spmm_csr(crow, col, val, H, out, relu_mask, r0, r1, lr)
    _count(2 if lr.numel() else 1)
    if out_dtype is not None and out_dtype != out.dtype:
        out = out.to(out_dtype)
    return out


def _bf16(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.bfloat16:
        return t
    raise TypeError(
        "the CUDA GEMM path takes bf16 activations (fp32 accumulate); got "
        f"{t.dtype}. Initialise with dtype=torch.bfloat16."
    )


def gemm(a, b, trans_a=False, trans_b=False, relu=False, out_dtype=None, variant: int = 0):
    C = _ext.load()
    st = status_buffer(a.device)
    max_stages, ctas = GEMM_VARIANTS[variant]
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
    out = torch.empty((a.shape[0], bt.shape[0]), dtype=out_dtype or a.dtype, device=a.device)
    C.gemm_nt(a, bt, out, bool(relu), st, max_stages, ctas)
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
