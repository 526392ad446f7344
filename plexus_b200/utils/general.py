"""Small utilities: seeding, padding, grid lookups, CSR statistics, timer report.

Reference: plexus/utils/general.py (set_seed :9-13, pad_dimension :20-23,
get_process_groups_info :28-49, analyze_csr_tensor :52-73, timer tree report
:93-154).
"""

from __future__ import annotations

import random
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..parallel.grid import get_grid
from ..parallel.sharding import pad_dimension  # noqa: F401  (re-exported)


def set_seed(seed: int = 0) -> None:
    """Give every rank the same seed for all host and device generators."""
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def get_process_groups_info(groups: Sequence[str]):
    """``(sizes, ranks, process_groups)`` for a tuple of distinct axis letters."""
    return get_grid().info(groups)


def analyze_csr_tensor(sparse_tensor) -> Tuple[int, float]:
    """Number of stored values and Frobenius norm of a CSR matrix."""
    values = sparse_tensor.values()
    nnz = values.numel()
    fro = torch.linalg.vector_norm(values.float()).item() if nnz else 0.0
    return nnz, fro


class color:
    """ANSI escape codes used by the timer tree."""

    PURPLE = "\033[95m"
    CYAN = "\033[96m"
    DARKCYAN = "\033[36m"
    BLUE = "\033[94m"
    GREEN = "\033[92m"
    YELLOW = "\033[93m"
    RED = "\033[91m"
    BOLD = "\033[1m"
    UNDERLINE = "\033[4m"
    END = "\033[0m"


class Node:
    """One line of the indented, coloured timer tree."""

    _palette = (color.PURPLE, color.GREEN, color.CYAN, color.RED)

    def __init__(self, value):
        self.value = value
        self.children: List["Node"] = []

    def add_children(self, child: "Node") -> None:
        self.children.append(child)

    def __str__(self, level: int = 0) -> str:
        c = self._palette[level % len(self._palette)]
        text = "\t" * level + "|--" + f"{c} {repr(self.value)} {color.END}" + "\n"
        return text + "".join(ch.__str__(level + 1) for ch in self.children)

    def __repr__(self) -> str:
        return f"\n{self.value}"


def reduce_timer_data(times: Dict[Tuple[str, ...], float]):
    """Max and mean over ranks of each timer key.  Returns {key: (max, avg)} on rank 0.

    All keys are reduced with two collectives (MAX and SUM over one vector)
    instead of two per key.
    """
    keys = sorted(times.keys(), key=lambda k: (len(k), k))
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return {k: (times[k], times[k]) for k in keys}
    use_cuda = dist.get_backend() == "nccl"
    dev = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    vec = torch.tensor([times[k] for k in keys], dtype=torch.float64, device=dev)
    mx, sm = vec.clone(), vec.clone()
    dist.reduce(mx, dst=0, op=dist.ReduceOp.MAX)
    dist.reduce(sm, dst=0, op=dist.ReduceOp.SUM)
    if dist.get_rank() != 0:
        return {}
    sm = sm / dist.get_world_size()
    return {k: (mx[i].item(), sm[i].item()) for i, k in enumerate(keys)}


def format_timer_tree(reduced) -> str:
    """Tree text with ``name | Max Time | Avg Time | Load Imbalance`` per region."""
    heads, nodes = [], {}
    for key in sorted(reduced.keys(), key=len):
        mx, avg = reduced[key]
        imb = mx / avg if avg > 0 else 1.0
        node = Node(
            f"{key[-1]} | Max Time: {mx:.3f} ms | Avg Time: {avg:.3f} ms | "
            f"Load Imbalance: {imb:.3f}"
        )
        nodes[key] = node
        if len(key) > 1 and key[:-1] in nodes:
            nodes[key[:-1]].add_children(node)
        else:
            heads.append(node)
    return "\n".join(str(h) for h in heads)


def print_axonn_timer_data(times) -> None:
    """Reduce the timer totals over ranks and print the region tree on rank 0."""
    reduced = reduce_timer_data(times)
    is_root = not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
    if is_root:
        print(format_timer_tree(reduced))


print_timer_data = print_axonn_timer_data
