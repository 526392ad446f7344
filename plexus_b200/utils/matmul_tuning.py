"""Dense GEMM entry point with optional per-site tuning.

``tuned_matmul(A, B, name)`` multiplies through :func:`plexus_b200.ops.gemm`.
With ``tune_gemms`` enabled, the first call for a given site name times a set
of candidate variants (5 warm-up + 20 timed runs each) and caches the fastest
one in ``matmul_to_index[name]``:

* on CPU tensors the candidates are the eight operand-layout / transposed-
  product variants the reference tunes over (reference:
  plexus/utils/matmul_tuning.py:55-74);
* on CUDA tensors the candidates are launch shapes of the tcgen05 GEMM
  (pipeline depth and CTAs per SM), see ``ops.cuda.GEMM_VARIANTS``.
"""

from __future__ import annotations

import time
from functools import partial

import torch

from .. import ops, runtime


def time_gpu(op, warmup: int = 5, trials: int = 20) -> float:
    """Mean seconds per call of ``op`` (device-synchronised when CUDA is in use)."""
    for _ in range(warmup):
        op()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(trials):
            op()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) * 1e-3 / trials
    t0 = time.perf_counter()
    for _ in range(trials):
        op()
    return (time.perf_counter() - t0) / trials


def matmul(A, B, change_layout, transpose=False):
    """``A @ B`` computed as ``(B^T A^T)^T`` when ``transpose``, with optional
    column-major copies of the operands (``change_layout[i]``)."""
    if transpose:
        A, B = B.t(), A.t()
    A = A.t().contiguous().t() if change_layout[0] else A.contiguous()
    B = B.t().contiguous().t() if change_layout[1] else B.contiguous()
    C = torch.mm(A, B)
    return C.t().contiguous() if transpose else C


# candidate configurations tried when tuning on CPU tensors
transpose_orders = [False] * 4 + [True] * 4
change_layouts = [(False, False), (True, False), (False, True), (True, True)] * 2

# cached best configuration per GEMM site
matmul_to_index = dict()


def _cpu_variant(A, B, idx, trans_a, trans_b, relu, out_dtype):
    x = A.t() if trans_a else A
    y = B.t() if trans_b else B
    from ..ops.reference import _acc

    x, y = _acc(x), _acc(y)
    if x.dtype != y.dtype:
        y = y.to(x.dtype)
    out = matmul(x, y, change_layouts[idx], transpose_orders[idx])
    if relu:
        out = torch.relu(out)
    return out.to(out_dtype or A.dtype)


def tuned_matmul(A, B, matmul_name, trans_a=False, trans_b=False, relu=False, out_dtype=None, relu_mask=None):
    """``op(A) @ op(B)``; tunes and caches the variant per ``matmul_name`` if enabled."""
    if not runtime.flags.tune_gemm:
        return ops.gemm(A, B, trans_a=trans_a, trans_b=trans_b, relu=relu, out_dtype=out_dtype,
                        relu_mask=relu_mask)

    if A.is_cuda:
        from ..ops import cuda as opc

        run = lambda i: opc.gemm(A, B, trans_a=trans_a, trans_b=trans_b, relu=relu,
                                 out_dtype=out_dtype, variant=i, relu_mask=relu_mask)
        n_variants = len(opc.GEMM_VARIANTS)
    else:
        def run(i):
            out = _cpu_variant(A, B, i, trans_a, trans_b, relu, out_dtype)
            return out if relu_mask is None else ops.relu_backward(out, relu_mask)
        n_variants = len(transpose_orders)

    if matmul_name not in matmul_to_index:
        best, best_t = 0, None
        for i in range(n_variants):
            t = time_gpu(partial(run, i))
            if best_t is None or t < best_t:
                best, best_t = i, t
        matmul_to_index[matmul_name] = best
    return run(matmul_to_index[matmul_name])
