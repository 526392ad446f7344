"""SpMM compute model: ranks grids by sparse work and operand aspect ratio.

``cost = c0*sqrt(F) + c1*sqrt(F)*fwd_pen + c2*sqrt(F)*bwd_pen`` with
``F = sum_l NNZ*D_l/(x*y*z)`` and penalties that grow when the dense operand of
the forward (``A.H``: ``N/outer`` rows by ``D/inner`` columns) or backward
(``A^T.gradAGG``: ``N/depth`` by ``D/inner``) SpMM becomes tall and skinny
(reference: performance/comp_model.py:27-64).

``spmm_time_b200`` is the bandwidth model used for this framework's own SpMM:
gathered feature rows dominate, ``bytes = nnz*(D*2 + 8) + rows*D*2``.
"""

from __future__ import annotations

from .common import split_into_three_powers_of_two  # noqa: F401


def comp_model(N, NNZ, G, D_list, coef=[1, 1, 1]):
    """Estimated SpMM cost per grid, ascending.  ``D_list`` excludes the class count."""
    costs = {}
    for x, y, z in split_into_three_powers_of_two(G):
        # per layer: outer, depth, inner sizes are ring[i], ring[i+1], ring[i+2]
        ring = (x, z, y)
        flops = fwd = bwd = 0.0
        for i, D in enumerate(D_list):
            outer, depth, inner = ring[i % 3], ring[(i + 1) % 3], ring[(i + 2) % 3]
            flops += NNZ * D / (outer * depth * inner)
            fwd += (N * inner) / (D * outer)
            bwd += (N * inner) / (D * depth)
        root = flops**0.5
        costs[(x, y, z)] = coef[0] * root + coef[1] * root * fwd + coef[2] * root * bwd
    return dict(sorted(costs.items(), key=lambda kv: kv[1]))


def spmm_time_b200(nnz, rows, D, hbm_gbs=6555.0, l2_hit=0.3, elem_bytes=2):
    """Milliseconds for one ``rows x *`` CSR SpMM of width ``D`` on one B200."""
    gathered = nnz * D * elem_bytes * (1.0 - l2_hit)
    meta = nnz * 8 + rows * 4
    out = rows * D * elem_bytes
    return (gathered + meta + out) / (hbm_gbs * 1e9) * 1e3
