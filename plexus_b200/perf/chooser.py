"""Pick the grid shape from the three cost models.

Grids whose estimated memory exceeds the device are dropped; the rest are
ranked by estimated communication time plus the bandwidth-model SpMM time on
this machine.
"""

from __future__ import annotations

from typing import List, Tuple

from .comm_model import compute_config_costs, load_measured_peaks
from .comp_model import spmm_time_b200
from .common import DEPTH, INNER, OUTER, split_into_three_powers_of_two
from .mem_model import compute_config_mem_b200


def choose_grid(G: int, N: int, NNZ: int, D_list: List[int], machine: str = "b200_nvl8",
                mem_limit_gb: float = 170.0) -> List[Tuple[int, int, int]]:
    """Grids ordered best first."""
    comm = compute_config_costs(G, N, D_list, "v3", machine)
    mem = compute_config_mem_b200(G, N, NNZ, D_list)
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
