"""Index arithmetic for sharding matrices over the grid.

All sizes are padded up to divisibility first; a rank's shard is the
contiguous block selected by its coordinate along the sharding axis.
"""

from __future__ import annotations

from typing import Tuple

import torch

from .grid import group_rank, group_size


def pad_dimension(dim_value: int, num_gpus: int, second_num_gpus: int = 1) -> int:
    """Smallest value >= ``dim_value`` divisible by ``num_gpus * second_num_gpus``.

    Reference: plexus/utils/general.py:20-23.
    """
    m = num_gpus * second_num_gpus
    return ((dim_value + m - 1) // m) * m


def padded_channels(channels: int, split: int, extra: int = 1, align: int = 1) -> int:
    """Pad a channel count so it splits in ``split`` blocks whose size is a
    multiple of both ``extra`` (a second sharding factor) and ``align``."""
    import math

    return pad_dimension(channels, split, math.lcm(max(1, extra), max(1, align)))


def block_range(total: int, parts: int, index: int) -> Tuple[int, int]:
    """[start, stop) of block ``index`` when ``total`` (padded) is split in ``parts``."""
    step = pad_dimension(total, parts) // parts
    return index * step, (index + 1) * step


def shard_2d(
    full: torch.Tensor, row_parts: int, row_index: int, col_parts: int, col_index: int
) -> torch.Tensor:
    """Block (row_index, col_index) of ``full`` after zero-padding to divisibility."""
    R = pad_dimension(full.shape[0], row_parts)
    C = pad_dimension(full.shape[1], col_parts)
    if (R, C) != tuple(full.shape):
        full = torch.nn.functional.pad(full, (0, C - full.shape[1], 0, R - full.shape[0]))
    r0, r1 = row_index * (R // row_parts), (row_index + 1) * (R // row_parts)
    c0, c1 = col_index * (C // col_parts), (col_index + 1) * (C // col_parts)
    return full[r0:r1, c0:c1]


def depth_slice(flat: torch.Tensor, parts: int, index: int) -> torch.Tensor:
    """Contiguous 1/parts slice of a flat tensor (length must divide evenly)."""
    if flat.numel() % parts != 0:
        raise ValueError(f"cannot split {flat.numel()} elements in {parts} depth slices")
    n = flat.numel() // parts
    return flat[index * n : (index + 1) * n]


def extract_local_params_from_full_params(
    full_params: torch.Tensor, out_features_group, in_features_group, depth_group
) -> torch.Tensor:
    """Local flat shard of a 2-D parameter.

    The LAST dimension is split over ``in_features_group`` and the FIRST over
    ``out_features_group`` (the naming follows a ``(out, in)`` linear weight);
    the block is flattened row-major and the ``depth_group`` rank's contiguous
    1/p slice is returned.  Called with ``(inner, outer, depth)`` on an
    ``(in, out)`` GCN weight this yields rows by inner rank and columns by
    outer rank (reference call sites: plexus/gcn_conv.py:371-390).
    """
    rows_parts, rows_idx = group_size(out_features_group), group_rank(out_features_group)
    cols_parts, cols_idx = group_size(in_features_group), group_rank(in_features_group)
    block = shard_2d(full_params, rows_parts, rows_idx, cols_parts, cols_idx)
    flat = block.contiguous().reshape(-1)
    return depth_slice(flat, group_size(depth_group), group_rank(depth_group)).clone()
