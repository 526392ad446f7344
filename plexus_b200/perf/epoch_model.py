"""Epoch-time model of this framework on one NVSwitch box of B200s, per region.

The reference's three models (communication volume, SpMM shape penalty, memory; reference:
performance/comm_model.py, comp_model.py, mem_model.py) rank grids without predicting a time.
This model walks the same per-layer schedule the layers execute (``models/gcn_conv.py``) and prices
every kernel and collective with constants measured on B200 (CUDA events, bf16):

* SpMM: ``rows * 200 ps + nnz * (9 ps + 0.073 ps per byte of a gathered row)`` - a least-squares fit
  through the measured 2.42 / 3.64 / 5.9 ms of the 123.7M-nonzero, 2.45M-row product at 48 / 104 / 256
  columns, the 1.42 ms of a 25M-nonzero, 1M-row product at 256 columns and the measured epochs below
  (per-row set-up and store, issue-bound cost per nonzero, L2-assisted 13.7 TB/s gather);
* tcgen05 GEMMs: operand + result bytes at 0.85 of the measured HBM copy bandwidth;
* fused all-reduce on a 2-rank axis: the push overlaps the compute kernel
  (``max(compute, bytes / 680 GB/s)``), the slot-reduce kernel moves 3 x message bytes through HBM;
* larger axes: segment reduce inside the switch after the compute kernel - ``(1 + 1/p)`` x message
  bytes per port at the measured 583 GB/s plus the copy out of the symmetric buffer (2 x message
  bytes through HBM) and two barriers; messages up to 1 MiB use the one-shot push (latency only);
* all-gather: ``(p-1)/p`` of the gathered bytes at the push rate plus the landing copy;
* cross-entropy and Adam: measured cost per element;
* every collective pays a launch + flag latency;
* every kernel launch pays a gap of 20 us (dependent launches do not start back to back; the small
  ATen ops between the kernels sit in there too): 0.7 ms of a 30 ms single-GPU epoch.

``predict_epoch_ms`` returns the regions and their sum; ``tests/test_perf_models.py`` pins it to the
measured epochs (29.9 ms on 1 GPU; 21.2 / 21.5 / 22.8 on the three 2-GPU grids; 14.65 / 15.53 on
2x2x1 / 2x1x2; 12.0 on 4x2x1) within 5 %, to the measured order of the 2- and 4-GPU grids, and to
the four 8-GPU grids of the dense-degree graph (233K nodes, 115M nonzeros) within 25 %.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

from .comm_model import load_measured_peaks
from .common import DEPTH, INNER, OUTER, split_into_three_powers_of_two

SPMM_PS_PER_ROW = 200.0
SPMM_PS_PER_NNZ = 9.0
SPMM_PS_PER_BYTE = 0.073
GEMM_HBM_FRACTION = 0.85
PUSH_GBS = 680.0            # achieved rate of epilogue stores into a peer's memory
SWITCH_REDUCE_GBS = 583.0   # per port and direction in the segment reduce (multimem), 512 MB messages
SMALL_MESSAGE_BYTES = 1 << 20
COLLECTIVE_LATENCY_MS = 0.02
XENT_PS_PER_ELEM = 2.8      # 0.33 ms for 2.45M rows x 48 classes
ADAM_PS_PER_ELEM = 4.4      # 1.12 ms for 255M bf16 elements with fp32 master and moments
LAUNCH_GAP_MS = 0.02        # per kernel launch: start-up gap of dependent launches + small glue ops
ELEM = 2                    # bf16


def _pad(v: int, m: int) -> int:
    return -(-v // m) * m


def _spmm_ms(nnz: float, row_elems: float, rows: float) -> float:
    return (rows * SPMM_PS_PER_ROW + nnz * (SPMM_PS_PER_NNZ + SPMM_PS_PER_BYTE * row_elems * ELEM)) * 1e-9


def _gemm_ms(m: float, k: float, n: float, hbm_gbs: float, out_bytes: int = ELEM) -> float:
    return (m * k * ELEM + k * n * ELEM + m * n * out_bytes) / (GEMM_HBM_FRACTION * hbm_gbs * 1e9) * 1e3


def _all_reduce_ms(p: int, elems: float, compute_ms: float, hbm_gbs: float) -> Tuple[float, float]:
    """``(time of compute + all-reduce, exposed communication)`` for a fused op on a ``p``-rank axis."""
    if p == 1:
        return compute_ms, 0.0
    nbytes = elems * ELEM
    if p == 2 or nbytes <= SMALL_MESSAGE_BYTES:
        link = (p - 1) * nbytes / (PUSH_GBS * 1e9) * 1e3
        reduce_ms = (p + 1) * nbytes / (hbm_gbs * 1e9) * 1e3
        total = max(compute_ms, link) + reduce_ms + COLLECTIVE_LATENCY_MS
    else:
        total = compute_ms + ((1 + 1 / p) * nbytes / (SWITCH_REDUCE_GBS * 1e9) + 2 * nbytes / (hbm_gbs * 1e9)) * 1e3 \
            + 2 * COLLECTIVE_LATENCY_MS
    return total, total - compute_ms


def _gather_ms(p: int, elems_total: float, hbm_gbs: float) -> float:
    if p == 1:
        return 0.0
    nbytes = elems_total * ELEM
    return ((p - 1) / p * nbytes / (PUSH_GBS * 1e9) + 2 * (p - 1) / p * nbytes / (hbm_gbs * 1e9)) * 1e3 \
        + COLLECTIVE_LATENCY_MS


def predict_epoch_ms(grid: Sequence[int], N: int, NNZ: int, D_list: List[int], align: int = 8,
                     hbm_gbs: float = None) -> Dict[str, float]:
    """Predicted milliseconds per region of one training epoch (forward, backward, loss, Adam)."""
    X, Y, Z = grid
    sizes = {"X": X, "Y": Y, "Z": Z}
    G = X * Y * Z
    hbm = hbm_gbs or load_measured_peaks().get("hbm_gbs", 6555.0)
    L = len(D_list) - 1
    r: Dict[str, float] = {"spmm": 0.0, "gemm": 0.0, "wgrad": 0.0, "exposed_comm": 0.0, "gather": 0.0,
                           "xent": 0.0, "adam": 0.0, "glue": 0.0}
    launches = 3  # cross-entropy (2) + Adam
    for i in range(L):
        po, pn, pd = sizes[OUTER[i % 3]], sizes[INNER[i % 3]], sizes[DEPTH[i % 3]]
        d_in = _pad(D_list[i], pn * (pd if i == 0 else 1) * align) / pn      # local input width
        d_out_full = _pad(D_list[i + 1], po * align)
        d_out = d_out_full / po                                              # local output width
        nnz = NNZ / (pd * po)
        rows_d, rows_o = N / pd, N / po
        combine_first = i > 0 and d_out_full < d_in
        # 2 SpMMs (items + long rows), 2-3 GEMMs with the weight re-layout, weight gradient (2 launches);
        # one more launch per collective that follows a kernel, two per gather
        launches += 4 + 3 + 1 + 2 + sum(1 for p_ in (po, pd, pn, po) if p_ > 1) + (2 if pd > 1 else 0)
        if i == 0:
            r["gather"] += _gather_ms(pd, rows_o * d_in, hbm)
        r["gather"] += 2 * (COLLECTIVE_LATENCY_MS if pd > 1 else 0.0)      # weight shards, fwd + bwd
        if not combine_first:
            for rows, p in ((rows_d, po), (rows_o, pd)):                      # A.H and A^T.gradAGG
                t = _spmm_ms(nnz, d_in, rows)
                total, exposed = _all_reduce_ms(p, rows * d_in, t, hbm)
                r["spmm"] += t
                r["exposed_comm"] += exposed
            t = _gemm_ms(rows_d, d_in, d_out, hbm)                            # OUT = AGG.W
            total, exposed = _all_reduce_ms(pn, rows_d * d_out, t, hbm)
            r["gemm"] += t
            r["exposed_comm"] += exposed
            t = _gemm_ms(rows_d, d_out, d_in, hbm)                            # gradAGG = gradOUT.W^T
            total, exposed = _all_reduce_ms(po, rows_d * d_in, t, hbm)
            r["gemm"] += t
            r["exposed_comm"] += exposed
            r["wgrad"] += _gemm_ms(rows_d, d_in, 0, hbm) + _gemm_ms(rows_d, d_out, 0, hbm)
        else:
            t = _gemm_ms(rows_o, d_in, d_out_full, hbm)                       # T = H.W
            total, exposed = _all_reduce_ms(pn, rows_o * d_out_full, t, hbm)
            r["gemm"] += t
            r["exposed_comm"] += exposed
            for rows, p in ((rows_d, po), (rows_o, pd)):                      # A.T and A^T.gradU
                t = _spmm_ms(nnz, d_out_full, rows)
                total, exposed = _all_reduce_ms(p, rows * d_out_full, t, hbm)
                r["spmm"] += t
                r["exposed_comm"] += exposed
            r["gather"] += _gather_ms(po, rows_d * d_out_full, hbm)           # gradOUT column blocks
            r["gemm"] += _gemm_ms(rows_o, d_out_full, d_in, hbm)              # gradH = gradT.W^T
            r["wgrad"] += _gemm_ms(rows_o, d_in, 0, hbm) + _gemm_ms(rows_o, d_out_full, 0, hbm)
        if pd > 1 or (combine_first and po > 1):
            r["exposed_comm"] += COLLECTIVE_LATENCY_MS                        # weight-gradient reduction
    # loss on the last layer's output layout
    po, pd = sizes[OUTER[(L - 1) % 3]], sizes[DEPTH[(L - 1) % 3]]
    c_local = _pad(D_list[-1], po * align) / po
    r["xent"] = (N / pd) * c_local * XENT_PS_PER_ELEM * 1e-9 + (3 * COLLECTIVE_LATENCY_MS if po > 1 else 0.0) \
        + (COLLECTIVE_LATENCY_MS if pd > 1 else 0.0)
    # Adam over the flat feature shard and the weight shards
    feat = N * _pad(D_list[0], Y * Z * align) / G
    weights = sum(D_list[i] * D_list[i + 1] for i in range(L)) / G
    r["adam"] = (feat + weights) * ADAM_PS_PER_ELEM * 1e-9 + 0.01
    r["glue"] = launches * LAUNCH_GAP_MS
    r["total"] = sum(r.values())
    return r


def rank_grids(G: int, N: int, NNZ: int, D_list: List[int]) -> List[Tuple[float, Tuple[int, int, int]]]:
    """``[(predicted epoch ms, grid)]`` for every power-of-two grid of ``G`` ranks, best first."""
    scored = [(predict_epoch_ms(g, N, NNZ, D_list)["total"], g) for g in split_into_three_powers_of_two(G)]
    return sorted(scored)
