"""Pick the grid shape from the cost models.

Grids whose estimated memory exceeds the device are dropped.  ``model="epoch"`` (the default on
``b200_nvl8``) orders the rest by the per-region epoch-time model of ``perf/epoch_model.py``, which
prices every kernel and collective of the executed schedule with measured constants; on 2 GPUs its
order 1x2x1 < 2x1x1 < 1x1x2 is the measured one (21.2 / 21.5 / 22.8 ms on the 2.45M-node graph).
``model="volume"`` orders them by estimated communication time plus the bandwidth-model SpMM time,
the reference's way of combining its models (it puts 1x1x2 first there).
"""

from __future__ import annotations

from typing import List, Tuple

from .comm_model import compute_config_costs, load_measured_peaks
from .comp_model import spmm_time_b200
from .common import DEPTH, INNER, OUTER, split_into_three_powers_of_two
from .mem_model import compute_config_mem_b200


def _message_limit() -> int:
    """The row-block limit of the fused collectives (``PLEXUS_MAX_MESSAGE_BYTES``, default 2 GiB): it
    bounds the peer-memory workspaces the memory model counts."""
    import os

    return int(os.environ.get("PLEXUS_MAX_MESSAGE_BYTES", str(2 << 30)))


def choose_grid(G: int, N: int, NNZ: int, D_list: List[int], machine: str = "b200_nvl8",
                mem_limit_gb: float = 170.0, model: str = "epoch") -> List[Tuple[int, int, int]]:
    """Grids ordered best first.  If no grid fits the memory limit, the one that needs the least
    memory comes back alone (lower ``PLEXUS_MAX_MESSAGE_BYTES`` to shrink the workspaces)."""
    mem = compute_config_mem_b200(G, N, NNZ, D_list, max_message_bytes=_message_limit())
    if not any(v <= mem_limit_gb for v in mem.values()):
        k = min(mem, key=mem.get)  # "X{X}Y{Y}Z{Z}"
        x, rest = k[1:].split("Y")
        y, z = rest.split("Z")
        return [(int(x), int(y), int(z))]
    if machine == "b200_nvl8" and model == "epoch":
        from .epoch_model import predict_epoch_ms

        fits = [g for g in split_into_three_powers_of_two(G) if mem[f"X{g[0]}Y{g[1]}Z{g[2]}"] <= mem_limit_gb]
        ranked = sorted((predict_epoch_ms(g, N, NNZ, D_list)["total"], g) for g in fits)
        return [g for _, g in ranked]
    comm = compute_config_costs(G, N, D_list, "v3", machine)
    hbm = load_measured_peaks().get("hbm_gbs", 6555.0)
    scored = []
    for X, Y, Z in split_into_three_powers_of_two(G):
        sizes = {"X": X, "Y": Y, "Z": Z}
        if mem[f"X{X}Y{Y}Z{Z}"] > mem_limit_gb:
            continue
        spmm = 0.0
        for i in range(len(D_list) - 1):
            o, n, d = sizes[OUTER[i % 3]], sizes[INNER[i % 3]], sizes[DEPTH[i % 3]]
            # forward A.H and backward A^T.gradAGG have the same nnz and width
            spmm += 2 * spmm_time_b200(NNZ / (d * o), N / d, D_list[i] / n, hbm)
        scored.append((comm[(X, Y, Z)] + spmm, (X, Y, Z)))
    scored.sort()
    return [g for _, g in scored] or [(G, 1, 1)]
