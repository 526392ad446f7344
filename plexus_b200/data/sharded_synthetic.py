"""Seeded synthetic graphs whose shards are generated rank-locally.

For graphs whose global edge list does not fit one device (e.g. 111M nodes / 3.2B nonzeros: the
int64 COO list alone is 51 GB, its sort several times that) no process may hold the whole graph.
Every quantity of the synthetic pipeline is a pure function of a counter (edge number, node id,
feature index), so each rank streams over the raw edge numbers in chunks and keeps only what falls
into the blocks it needs:

* degree pass: rank ``k`` de-duplicates the edges whose row lies in stripe ``k`` of the node range
  and counts them; one all-gather gives every rank the full degree vector (4 bytes per node);
* block pass: one stream over the raw edges serves all requested blocks at once.  An edge
  ``(r, c)`` of the symmetrised graph lands at ``(inv_P[r], inv_P2[c])`` in version 0
  (``P A P2^T``) and at ``(inv_P2[r], inv_P[c])`` in version 1; entries inside a requested block
  are kept as ``row * ncols + col`` keys, de-duplicated at the end, and their values
  ``d_r^-1/2 d_c^-1/2`` are computed from the keys alone;
* features, labels and masks of the permuted node order are hashed directly for the requested
  rows.

The graph is defined as "raw edges ``0 .. num_raw_edges-1`` of the generator, self loops removed,
symmetrised, de-duplicated, plus one self loop per node"; the resulting shards are identical to
what :func:`synthetic_graph_from_raw_edges` + ``preprocess_data`` + ``DataLoader`` produce from the
global edge list (checked in the tests on small graphs).

The reference has no generator; it preprocesses downloaded datasets on one host
(plexus/utils/dataset.py:29-249) and its loader slices a global edge list per rank
(plexus/utils/dataloader.py:327-375).
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import graph_ops
from .container import Data
from .synthetic import _MASK63, hash_stream, normal01, rmat_edges, uniform01, uniform_edges

Block = Tuple[int, int, int, int, int]  # (version, r0, r1, c0, c1)


def raw_undirected_keys(num_nodes: int, num_raw_edges: int, seed: int = 0, kind: str = "rmat",
                        device="cpu", chunk: int = 1 << 24, **rmat_kw) -> torch.Tensor:
    """Sorted unique ``lo * N + hi`` keys (lo < hi) of raw edges ``0 .. num_raw_edges-1``."""
    gen = rmat_edges if kind == "rmat" else uniform_edges
    kw = rmat_kw if kind == "rmat" else {}
    parts = []
    for first in range(0, num_raw_edges, chunk):
        n = min(chunk, num_raw_edges - first)
        r, c = gen(num_nodes, first, n, seed=seed, device=device, **kw)
        lo, hi = torch.minimum(r, c), torch.maximum(r, c)
        parts.append(torch.unique((lo * num_nodes + hi)[lo != hi]))
    if not parts:
        return torch.empty(0, dtype=torch.int64, device=device)
    return torch.unique(torch.cat(parts))


def synthetic_graph_from_raw_edges(num_nodes: int, num_raw_edges: int, num_features: int, num_classes: int,
                                   seed: int = 0, kind: str = "rmat", device="cpu", **rmat_kw):
    """Global (single-process) form of the graph :class:`ShardedSyntheticGraph` describes."""
    from .synthetic import synthetic_features, synthetic_labels

    keys = raw_undirected_keys(num_nodes, num_raw_edges, seed, kind, device, **rmat_kw)
    edge_index = graph_ops.symmetrize_with_self_loops(keys, num_nodes)
    data = Data(x=synthetic_features(num_nodes, num_features, seed, device=device),
                y=synthetic_labels(num_nodes, num_classes, seed, device=device),
                edge_index=edge_index, edge_weight=graph_ops.gcn_normalize(edge_index, num_nodes))
    data.symmetric = True
    u = uniform01(seed, 4000, torch.arange(num_nodes, dtype=torch.int64, device=device))
    data.train_mask, data.val_mask, data.test_mask = u < 0.5, (u >= 0.5) & (u < 0.75), u >= 0.75
    return data, num_classes


class ShardedSyntheticGraph:
    """Source object for ``DataLoader(source=...)``: symmetric, normalised, double-permuted."""

    symmetric = True
    double_perm = True

    def __init__(self, num_nodes: int, num_raw_edges: int, num_features: int, num_classes: int, seed: int = 0,
                 kind: str = "rmat", device=None, chunk: int = 1 << 24, group=None, **rmat_kw):
        self.num_nodes, self.num_raw_edges = int(num_nodes), int(num_raw_edges)
        self.num_features, self.num_classes = int(num_features), int(num_classes)
        self.seed, self.kind, self.chunk, self.group = seed, kind, int(chunk), group
        self.rmat_kw = rmat_kw if kind == "rmat" else {}
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        # the same two permutations preprocess_data draws for this seed
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed)
        self.perm = [torch.randperm(self.num_nodes, generator=gen).to(self.device),
                     torch.randperm(self.num_nodes, generator=gen).to(self.device)]
        self.inv = [graph_ops.inverse_permutation(p) for p in self.perm]
        self._dinv: Optional[torch.Tensor] = None
        self.nnz_total: Optional[int] = None

    # ------------------------------------------------------------------ raw edge stream
    def _chunks(self):
        gen = rmat_edges if self.kind == "rmat" else uniform_edges
        for first in range(0, self.num_raw_edges, self.chunk):
            n = min(self.chunk, self.num_raw_edges - first)
            r, c = gen(self.num_nodes, first, n, seed=self.seed, device=self.device, **self.rmat_kw)
            keep = r != c
            yield r[keep], c[keep]

    # ------------------------------------------------------------------ degrees
    def _world(self):
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(self.group), dist.get_world_size(self.group)
        return 0, 1

    def inverse_sqrt_degree(self) -> torch.Tensor:
        """``d^-1/2`` for every node, ``d`` = distinct neighbours + 1 (the self loop)."""
        if self._dinv is not None:
            return self._dinv
        N = self.num_nodes
        rank, world = self._world()
        stripe = (N + world - 1) // world
        s0, s1 = min(rank * stripe, N), min((rank + 1) * stripe, N)
        parts: List[torch.Tensor] = []
        pending = 0
        for r, c in self._chunks():
            # both directions of every undirected edge whose row lies in this rank's stripe
            for a, b in ((r, c), (c, r)):
                m = (a >= s0) & (a < s1)
                parts.append((a[m] - s0) * N + b[m])
                pending += int(parts[-1].numel())
            if pending > 8 * self.chunk:  # bound the memory of the duplicates
                parts = [torch.unique(torch.cat(parts))]
                pending = int(parts[0].numel())
        keys = torch.unique(torch.cat(parts)) if parts else torch.empty(0, dtype=torch.int64, device=self.device)
        counts = torch.zeros(stripe, dtype=torch.float32, device=self.device)
        if keys.numel():
            rows = torch.div(keys, N, rounding_mode="floor")
            counts += torch.bincount(rows, minlength=stripe).to(torch.float32)
        counts += 1.0  # self loop
        if world > 1:
            allc = torch.empty(world * stripe, dtype=torch.float32, device=self.device)
            dist.all_gather_into_tensor(allc, counts, group=self.group)
            counts = allc
            nnz = torch.tensor([keys.numel()], dtype=torch.int64, device=self.device)
            dist.all_reduce(nnz, group=self.group)
            self.nnz_total = int(nnz.item()) + N
        else:
            self.nnz_total = int(keys.numel()) + N
        self._dinv = counts[:N].pow(-0.5)
        return self._dinv

    # ------------------------------------------------------------------ adjacency blocks
    def build_blocks(self, blocks: Sequence[Block]) -> Dict[Block, torch.Tensor]:
        """CSR tensors (int32 indices, fp32 values) of the requested ``(version, r0, r1, c0, c1)``
        blocks of ``P A P2^T`` (version 0) / ``P2 A P^T`` (version 1), from ONE pass over the raw edges."""
        blocks = list(dict.fromkeys(blocks))
        dinv = self.inverse_sqrt_degree()
        kept: Dict[Block, List[torch.Tensor]] = {b: [] for b in blocks}

        def scatter(version, rows, cols):
            # rows / cols are permuted coordinates of this version
            for b in blocks:
                v, r0, r1, c0, c1 = b
                if v != version:
                    continue
                m = (rows >= r0) & (rows < r1) & (cols >= c0) & (cols < c1)
                if bool(m.any()):
                    kept[b].append((rows[m] - r0) * (c1 - c0) + (cols[m] - c0))

        versions = sorted({b[0] for b in blocks})
        for r, c in self._chunks():
            for v in versions:
                ir, ic = self.inv[v], self.inv[1 - v]  # version 0: rows by P, columns by P2
                pr, pc = ir[r], ic[c]      # edge (r, c)
                qr, qc = ir[c], ic[r]      # edge (c, r)
                scatter(v, pr, pc)
                scatter(v, qr, qc)
        # self loops: node i sits at (inv_row[i], inv_col[i])
        loops = torch.arange(self.num_nodes, dtype=torch.int64, device=self.device)
        for v in versions:
            scatter(v, self.inv[v][loops], self.inv[1 - v][loops])

        out: Dict[Block, torch.Tensor] = {}
        for b in blocks:
            v, r0, r1, c0, c1 = b
            ncols = c1 - c0
            keys = (torch.unique(torch.cat(kept[b])) if kept[b]
                    else torch.empty(0, dtype=torch.int64, device=self.device))
            kept[b] = []
            rows = torch.div(keys, ncols, rounding_mode="floor")
            cols = keys - rows * ncols
            # value from the original endpoints of the entry
            orig_r = self.perm[v][rows + r0]
            orig_c = self.perm[1 - v][cols + c0]
            vals = (dinv[orig_r] * dinv[orig_c]).to(torch.float32)
            del orig_r, orig_c
            crow, col, val = graph_ops.coo_to_csr(rows, cols, vals, r1 - r0, ncols, assume_sorted=True)
            out[b] = graph_ops.csr_tensor(crow, col, val, (r1 - r0, ncols))
        return out

    # ------------------------------------------------------------------ node data
    def feature_block(self, r0: int, r1: int, c0: int, c1: int, dtype=torch.float32,
                      chunk_rows: int = 1 << 18) -> torch.Tensor:
        """Rows ``[r0, r1)`` x columns ``[c0, c1)`` of the permuted feature matrix ``x[P2]``; rows past
        the node count and columns past the feature count are zero."""
        N, F = self.num_nodes, self.num_features
        out = torch.zeros((r1 - r0, c1 - c0), dtype=dtype, device=self.device)
        rr1, cc1 = min(r1, N), min(c1, F)
        if rr1 <= r0 or cc1 <= c0:
            return out
        cols = torch.arange(c0, cc1, dtype=torch.int64, device=self.device)
        for a in range(r0, rr1, chunk_rows):
            b = min(rr1, a + chunk_rows)
            orig = self.perm[1][a:b]
            idx = orig[:, None] * F + cols[None, :]
            out[a - r0 : b - r0, : cc1 - c0] = normal01(self.seed, 5000, idx.reshape(-1), torch.float32).view(
                b - a, cc1 - c0).to(dtype)
        return out

    def labels(self, version: int, r0: int, r1: int) -> torch.Tensor:
        """``y[P]`` (version 0) or ``y[P2]`` (version 1) for rows ``[r0, min(r1, N))``."""
        orig = self.perm[version][r0 : min(r1, self.num_nodes)]
        return (hash_stream(self.seed, 6000, orig) & _MASK63) % self.num_classes

    def mask(self, name: str, version: int, r0: int, r1: int) -> torch.Tensor:
        orig = self.perm[version][r0 : min(r1, self.num_nodes)]
        u = uniform01(self.seed, 4000, orig)
        if name == "train_mask":
            return u < 0.5
        if name == "val_mask":
            return (u >= 0.5) & (u < 0.75)
        if name == "test_mask":
            return u >= 0.75
        raise KeyError(name)


def write_partition_tree(source: ShardedSyntheticGraph, num_partitions: int, output_dir: str,
                         blocks_per_pass: int = 8) -> None:
    """Write the ``p x p`` partition tree the loader reads (``metadata.pt``, ``edge_index/{0,1}/i_j.pt``
    with global indices, ``input_features/i_j.pt``, ``output_labels/{0,1}/i.pt``, ``extra.pt``) straight
    from the generator: no process builds the global graph.  With a process group the ranks split the
    blocks between them (rank ``r`` writes blocks ``r, r + world, ...``), ``blocks_per_pass`` block
    positions (both permutation versions of each) are produced by one pass over the raw edge stream.

    Same files as ``utils.dataset.partition_graph_2d`` writes from a processed file
    (reference: plexus/utils/dataset.py:370-566).
    """
    import os

    from ..parallel.sharding import pad_dimension
    from ..utils.dataset import _atomic_save

    p = int(num_partitions)
    N, F = source.num_nodes, source.num_features
    chunk_n, chunk_f = pad_dimension(N, p) // p, pad_dimension(F, p) // p
    rank, world = source._world()
    for sub in ("edge_index/0", "edge_index/1", "input_features", "output_labels/0", "output_labels/1"):
        os.makedirs(os.path.join(output_dir, sub), exist_ok=True)
    mine = [(i, j) for k, (i, j) in enumerate((i, j) for i in range(p) for j in range(p)) if k % world == rank]
    source.inverse_sqrt_degree()  # collective: every rank takes part even if it writes no block
    for start in range(0, len(mine), blocks_per_pass):
        group = mine[start : start + blocks_per_pass]
        want = [(v, i * chunk_n, (i + 1) * chunk_n, j * chunk_n, (j + 1) * chunk_n) for i, j in group for v in (0, 1)]
        built = source.build_blocks(want)
        for i, j in group:
            for v in (0, 1):
                A = built[(v, i * chunk_n, (i + 1) * chunk_n, j * chunk_n, (j + 1) * chunk_n)]
                crow, col, val = A.crow_indices().to(torch.int64), A.col_indices().to(torch.int64), A.values()
                rows = torch.repeat_interleave(torch.arange(crow.numel() - 1, device=crow.device), crow[1:] - crow[:-1])
                ei = torch.stack([rows + i * chunk_n, col + j * chunk_n]).cpu()
                _atomic_save((ei, val.cpu()), os.path.join(output_dir, "edge_index", str(v), f"{i}_{j}.pt"))
            r0, r1 = i * chunk_n, min((i + 1) * chunk_n, N)
            f0, f1 = j * chunk_f, min((j + 1) * chunk_f, F)
            x = source.feature_block(r0, max(r0, r1), f0, max(f0, f1)).cpu()
            _atomic_save(x, os.path.join(output_dir, "input_features", f"{i}_{j}.pt"))
            if j == 0:
                for v in (0, 1):
                    _atomic_save(source.labels(v, r0, r1).cpu(),
                                 os.path.join(output_dir, "output_labels", str(v), f"{i}.pt"))
    if rank == 0:
        _atomic_save({"symmetric": True}, os.path.join(output_dir, "extra.pt"))
        _atomic_save((N, F, source.num_classes), os.path.join(output_dir, "metadata.pt"))
    if world > 1:
        dist.barrier(group=source.group)
