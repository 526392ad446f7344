"""Graph preprocessing primitives on COO edge lists (device-agnostic torch).

* self-loops + symmetric GCN normalisation ``D^-1/2 (A + I) D^-1/2``
  (what PyG's ``GCNNorm`` does in the reference, plexus/utils/dataset.py:101);
* vertex permutation as an index relabel.  The reference forms
  ``P A P2^T`` with sparse x sparse products (plexus/utils/dataset.py:136-198);
  the same matrix is obtained in O(E) by mapping ``row -> inv_perm[row]`` and
  ``col -> inv_perm2[col]``;
* COO -> CSR (sort + count + scan), CSR transpose, 2-D block extraction.

On a CUDA device the sort / scan calls run on the GPU; these are start-up
costs, not part of the training step.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch


def symmetrize_with_self_loops(keys: torch.Tensor, num_nodes: int) -> torch.Tensor:
    """``edge_index [2, E]`` (sorted by row, then col) from unique ``lo*N+hi`` keys, lo<hi."""
    lo = torch.div(keys, num_nodes, rounding_mode="floor")
    hi = keys - lo * num_nodes
    loops = torch.arange(num_nodes, dtype=torch.int64, device=keys.device)
    full = torch.cat([keys, hi * num_nodes + lo, loops * num_nodes + loops])
    del lo, hi
    full = torch.sort(full).values
    row = torch.div(full, num_nodes, rounding_mode="floor")
    col = full - row * num_nodes
    return torch.stack([row, col])


def add_remaining_self_loops(edge_index, edge_weight, num_nodes):
    """Drop existing self loops and add one of weight 1 per node."""
    keep = edge_index[0] != edge_index[1]
    loops = torch.arange(num_nodes, dtype=edge_index.dtype, device=edge_index.device)
    ei = torch.cat([edge_index[:, keep], torch.stack([loops, loops])], dim=1)
    if edge_weight is None:
        ew = torch.ones(ei.shape[1], dtype=torch.float32, device=ei.device)
    else:
        ew = torch.cat([edge_weight[keep], torch.ones(num_nodes, dtype=edge_weight.dtype, device=ei.device)])
    return ei, ew


def gcn_normalize(edge_index: torch.Tensor, num_nodes: int, edge_weight: Optional[torch.Tensor] = None):
    """Weights ``w_ij * d_i^-1/2 * d_j^-1/2`` with ``d`` the weighted in-degree (by column).

    ``edge_index`` must already contain the self loops.
    """
    if edge_index.is_cuda and edge_index.dtype == torch.int64 and edge_index.is_contiguous():
        from ..ops import _ext

        if _ext.available():
            w = None if edge_weight is None else edge_weight.float().contiguous()
            return _ext.load().gcn_norm(edge_index, w, num_nodes)
    if edge_weight is None:
        edge_weight = torch.ones(edge_index.shape[1], dtype=torch.float32, device=edge_index.device)
    deg = torch.zeros(num_nodes, dtype=torch.float32, device=edge_index.device)
    deg.scatter_add_(0, edge_index[1], edge_weight.float())
    dinv = deg.pow(-0.5)
    dinv[torch.isinf(dinv)] = 0.0
    return (dinv[edge_index[0]] * edge_weight.float() * dinv[edge_index[1]]).to(torch.float32)


def inverse_permutation(perm: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
    return inv


def permute_edges(edge_index, row_perm, col_perm, edge_weight=None, sort: bool = True):
    """Edge list of ``P_row A P_col^T`` where new row i is old row ``row_perm[i]``.

    Returns ``(edge_index, edge_weight)`` sorted by (row, col) when ``sort``.
    """
    inv_r = inverse_permutation(row_perm)
    inv_c = inv_r if col_perm is row_perm else inverse_permutation(col_perm)
    r = inv_r[edge_index[0]]
    c = inv_c[edge_index[1]]
    if sort:
        n = row_perm.numel()
        order = torch.argsort(r * n + c)
        r, c = r[order], c[order]
        if edge_weight is not None:
            edge_weight = edge_weight[order]
    return torch.stack([r, c]), edge_weight


def coo_to_csr(
    row: torch.Tensor,
    col: torch.Tensor,
    val: torch.Tensor,
    num_rows: int,
    num_cols: int,
    index_dtype=torch.int32,
    assume_sorted: bool = False,
):
    """``(crow, col, val)`` with columns ascending inside each row."""
    if (row.is_cuda and index_dtype == torch.int32 and val.dtype == torch.float32
            and 0 < row.numel() < 2**31 - 1 and not assume_sorted):
        from ..ops import _ext

        if _ext.available():
            # one radix sort of (row * ncols + col) keys, histogram and scan in the extension
            return _ext.load().coo_to_csr(row.to(torch.int64).contiguous(), col.to(torch.int64).contiguous(),
                                          val.contiguous(), num_rows, num_cols)
    if not assume_sorted and row.numel():
        order = torch.argsort(row.to(torch.int64) * num_cols + col.to(torch.int64))
        row, col, val = row[order], col[order], val[order]
    counts = torch.bincount(row, minlength=num_rows) if row.numel() else torch.zeros(
        num_rows, dtype=torch.int64, device=row.device
    )
    crow = torch.zeros(num_rows + 1, dtype=torch.int64, device=row.device)
    torch.cumsum(counts, 0, out=crow[1:])
    if row.numel() >= 2**31 - 1 and index_dtype == torch.int32:
        raise ValueError("shard has too many nonzeros for int32 row pointers")
    return crow.to(index_dtype), col.to(index_dtype), val


def csr_tensor(crow, col, val, shape):
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)
        return torch.sparse_csr_tensor(crow, col, val, size=tuple(shape), check_invariants=False)


def csr_transpose(A: torch.Tensor) -> torch.Tensor:
    """CSR of ``A^T`` by re-sorting the expanded coordinates."""
    crow, col, val = A.crow_indices(), A.col_indices(), A.values()
    nrows, ncols = A.shape
    counts = (crow[1:] - crow[:-1]).to(torch.int64)
    row = torch.repeat_interleave(
        torch.arange(nrows, dtype=torch.int64, device=crow.device), counts
    )
    c2, r2, v2 = coo_to_csr(col.to(torch.int64), row, val, ncols, nrows, index_dtype=crow.dtype)
    return csr_tensor(c2, r2, v2, (ncols, nrows))


def extract_block(
    edge_index: torch.Tensor,
    edge_weight: torch.Tensor,
    r0: int,
    r1: int,
    c0: int,
    c1: int,
    sorted_by_row: bool = False,
):
    """Edges inside ``[r0,r1) x [c0,c1)``, re-based to the block origin."""
    row, col = edge_index[0], edge_index[1]
    if sorted_by_row and row.numel():
        lo = int(torch.searchsorted(row, torch.tensor(r0, device=row.device, dtype=row.dtype)))
        hi = int(torch.searchsorted(row, torch.tensor(r1, device=row.device, dtype=row.dtype)))
        row, col, edge_weight = row[lo:hi], col[lo:hi], edge_weight[lo:hi]
        mask = (col >= c0) & (col < c1)
    else:
        mask = (row >= r0) & (row < r1) & (col >= c0) & (col < c1)
    return row[mask] - r0, col[mask] - c0, edge_weight[mask]


def block_nnz_counts(edge_index: torch.Tensor, num_nodes: int, parts: int) -> torch.Tensor:
    """nnz of each block of a ``parts x parts`` split (block size ``N // parts``, last takes the rest)."""
    size = max(1, num_nodes // parts)
    bi = torch.clamp(torch.div(edge_index[0], size, rounding_mode="floor"), max=parts - 1)
    bj = torch.clamp(torch.div(edge_index[1], size, rounding_mode="floor"), max=parts - 1)
    return torch.bincount(bi * parts + bj, minlength=parts * parts).view(parts, parts)
