"""Process grid for 3D tensor-parallel GCN training.

A job of ``G = X * Y * Z`` ranks is arranged as a 3D grid.  The rank order is
"Y fastest, then X, then Z": ``rank = z * (X * Y) + x * Y + y``.  Every rank
belongs to three *line groups*, one per axis (the ranks that differ from it
only in that coordinate).

Each GCN layer assigns the three axes the roles (outer, inner, depth) and the
assignment rotates with the layer index so that the output layout of one
layer is exactly the input layout of the next:

    layer % 3 == 0 -> (x, y, z)
    layer % 3 == 1 -> (z, x, y)
    layer % 3 == 2 -> (y, z, x)

This module replaces what the reference obtains from AxoNN's communication
handle (reference: plexus/plexus.py:35-41, plexus/utils/general.py:28-49,
plexus/gcn_conv.py:309-316).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

AXES = ("x", "y", "z")

# (outer, inner, depth) per layer index modulo 3.
_ROLE_ROTATION = (("x", "y", "z"), ("z", "x", "y"), ("y", "z", "x"))


def axis_roles(layer_num: int) -> Tuple[str, str, str]:
    """Axis letters playing (outer, inner, depth) at ``layer_num``."""
    return _ROLE_ROTATION[layer_num % 3]


def loss_axes(num_layers: int) -> Tuple[str, str]:
    """(row axis, class axis) of the logits produced by a ``num_layers`` GCN.

    The logits of the last layer ``L-1`` are laid out ``(N/depth) x (C/outer)``
    of that layer (reference: plexus/cross_entropy.py:24-31).
    """
    outer, _inner, depth = axis_roles(num_layers - 1)
    return depth, outer


def coords_of(rank: int, X: int, Y: int, Z: int) -> Tuple[int, int, int]:
    """(x, y, z) coordinates of ``rank``."""
    if not 0 <= rank < X * Y * Z:
        raise ValueError(f"rank {rank} outside a {X}x{Y}x{Z} grid")
    y = rank % Y
    x = (rank // Y) % X
    z = rank // (X * Y)
    return x, y, z


def rank_of(x: int, y: int, z: int, X: int, Y: int, Z: int) -> int:
    return z * (X * Y) + x * Y + y


def line_ranks(axis: str, x: int, y: int, z: int, X: int, Y: int, Z: int) -> List[int]:
    """Global ranks of the line through (x, y, z) along ``axis``, in axis order."""
    if axis == "x":
        return [rank_of(i, y, z, X, Y, Z) for i in range(X)]
    if axis == "y":
        return [rank_of(x, i, z, X, Y, Z) for i in range(Y)]
    if axis == "z":
        return [rank_of(x, y, i, X, Y, Z) for i in range(Z)]
    raise ValueError("A group can only be x, y, or z.")


@dataclass
class ProcessGrid:
    """The X x Y x Z grid as seen from one rank."""

    X: int
    Y: int
    Z: int
    rank: int
    world_size: int
    groups: Dict[str, Optional[object]] = field(default_factory=dict)
    lines: Dict[str, List[int]] = field(default_factory=dict)

    # --- construction -----------------------------------------------------
    @classmethod
    def build(
        cls,
        X: int = 1,
        Y: int = 1,
        Z: int = 1,
        rank: Optional[int] = None,
        world_size: Optional[int] = None,
        create_groups: bool = True,
    ) -> "ProcessGrid":
        """Build the grid; creates one process group per grid line.

        ``dist.new_group`` is a world-collective call, so every rank creates
        every line group in the same order and keeps only its own three.
        Axes of size 1 get no group (their collectives are no-ops).
        """
        if dist.is_available() and dist.is_initialized():
            rank = dist.get_rank() if rank is None else rank
            world_size = dist.get_world_size() if world_size is None else world_size
        else:
            rank = 0 if rank is None else rank
            world_size = X * Y * Z if world_size is None else world_size
        if X * Y * Z != world_size:
            raise ValueError(
                f"grid {X}x{Y}x{Z} = {X * Y * Z} ranks does not match world size {world_size}"
            )
        grid = cls(X=X, Y=Y, Z=Z, rank=rank, world_size=world_size)
        x, y, z = grid.coords
        for axis in AXES:
            grid.lines[axis] = line_ranks(axis, x, y, z, X, Y, Z)
            grid.groups[axis] = None
        if create_groups and dist.is_available() and dist.is_initialized() and world_size > 1:
            for axis in AXES:
                if grid.size(axis) == 1:
                    continue
                seen = set()
                for r in range(world_size):
                    rx, ry, rz = coords_of(r, X, Y, Z)
                    members = tuple(line_ranks(axis, rx, ry, rz, X, Y, Z))
                    if members in seen:
                        continue
                    seen.add(members)
                    pg = dist.new_group(ranks=list(members))
                    if rank in members:
                        grid.groups[axis] = pg
        return grid

    # --- queries ----------------------------------------------------------
    @property
    def coords(self) -> Tuple[int, int, int]:
        return coords_of(self.rank, self.X, self.Y, self.Z)

    def size(self, axis: str) -> int:
        return {"x": self.X, "y": self.Y, "z": self.Z}[axis.lower()]

    def coord(self, axis: str) -> int:
        x, y, z = self.coords
        return {"x": x, "y": y, "z": z}[axis.lower()]

    def group(self, axis: str):
        return self.groups.get(axis.lower())

    def roles(self, layer_num: int) -> "LayerRoles":
        o, i, d = axis_roles(layer_num)
        return LayerRoles(
            outer=o,
            inner=i,
            depth=d,
            outer_size=self.size(o),
            inner_size=self.size(i),
            depth_size=self.size(d),
            outer_rank=self.coord(o),
            inner_rank=self.coord(i),
            depth_rank=self.coord(d),
            outer_group=self.group(o),
            inner_group=self.group(i),
            depth_group=self.group(d),
        )

    def info(self, axes: Sequence[str]):
        """(sizes, ranks, groups) for the requested axis letters, in order."""
        axes = [a.lower() for a in axes]
        if len(set(axes)) != len(axes):
            raise AssertionError("Please input different groups.")
        for a in axes:
            if a not in AXES:
                raise ValueError("A group can only be x, y, or z.")
        return (
            [self.size(a) for a in axes],
            [self.coord(a) for a in axes],
            [self.group(a) for a in axes],
        )


@dataclass
class LayerRoles:
    outer: str
    inner: str
    depth: str
    outer_size: int
    inner_size: int
    depth_size: int
    outer_rank: int
    inner_rank: int
    depth_rank: int
    outer_group: object = None
    inner_group: object = None
    depth_group: object = None


class CommHandle:
    """Attribute view of the grid under the names AxoNN's handle exposes.

    Kept so code written against the reference's ``ax.comm_handle`` fields
    (reference: plexus/utils/general.py:36-46) keeps working.
    """

    def __init__(self, grid: ProcessGrid):
        self._grid = grid

    @property
    def G_intra_r(self):
        return self._grid.X

    @property
    def G_intra_c(self):
        return self._grid.Y

    @property
    def G_intra_d(self):
        return self._grid.Z

    @property
    def intra_layer_row_parallel_rank(self):
        return self._grid.coord("x")

    @property
    def intra_layer_column_parallel_rank(self):
        return self._grid.coord("y")

    @property
    def intra_layer_depth_parallel_rank(self):
        return self._grid.coord("z")

    @property
    def outer_intra_layer_parallel_group(self):
        return self._grid.group("x")

    @property
    def inner_intra_layer_parallel_group(self):
        return self._grid.group("y")

    @property
    def depth_intra_layer_parallel_group(self):
        return self._grid.group("z")


_GRID: Optional[ProcessGrid] = None


def set_grid(grid: Optional[ProcessGrid]) -> None:
    global _GRID
    _GRID = grid


def get_grid() -> ProcessGrid:
    if _GRID is None:
        raise RuntimeError("plexus_b200.init() has not been called")
    return _GRID


def grid_is_initialized() -> bool:
    return _GRID is not None


def group_size(group) -> int:
    """Size of a process group; ``None`` stands for a singleton axis."""
    if group is None:
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None:
        return 0
    return dist.get_rank(group)


def default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")
