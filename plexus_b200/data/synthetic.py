"""Seeded synthetic graphs (R-MAT and uniform), features and labels.

Everything is produced by a counter-based hash of ``(seed, stream, index)``
in 64-bit integer arithmetic, so

* the same seed gives the same graph on CPU and on GPU and for any number of
  ranks, and
* any contiguous range of edge indices can be generated on its own, which
  lets a rank generate only the chunk it is streaming through.

R-MAT picks one quadrant per bit level with probabilities (a, b, c, d); the
comparison is done on 16-bit integers so no floating-point rounding can make
devices disagree.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .container import Data

_MASK63 = (1 << 63) - 1
_GOLDEN = 0x9E3779B97F4A7C15 - (1 << 64)  # as signed int64
_M1 = 0xBF58476D1CE4E5B9 - (1 << 64)
_M2 = 0x94D049BB133111EB - (1 << 64)


def _lsr(x: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 values."""
    return (x >> n) & ((1 << (64 - n)) - 1)


def mix64(x: torch.Tensor) -> torch.Tensor:
    """SplitMix64 finaliser on int64 tensors (wrap-around arithmetic)."""
    x = x + _GOLDEN
    x = (x ^ _lsr(x, 30)) * _M1
    x = (x ^ _lsr(x, 27)) * _M2
    return x ^ _lsr(x, 31)


def hash_stream(seed: int, stream: int, index: torch.Tensor) -> torch.Tensor:
    """64 pseudo-random bits per element of ``index`` (int64)."""
    key = (seed * 0x632BE59BD9B4E019 + stream * 0xD1342543DE82EF95 + 0x2545F4914F6CDD1D) % (1 << 63)
    return mix64(mix64(index + key) ^ key)


def uniform01(seed: int, stream: int, index: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """Uniform [0, 1) from the top 24 bits of the hash."""
    bits = _lsr(hash_stream(seed, stream, index), 40)
    return bits.to(dtype) * (1.0 / (1 << 24))


def normal01(seed: int, stream: int, index: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """Standard normal by Box-Muller from two hashed uniforms."""
    u1 = uniform01(seed, stream, index, torch.float32).clamp_min(1.0 / (1 << 25))
    u2 = uniform01(seed, stream + 7919, index, torch.float32)
    z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * math.pi) * u2)
    return z.to(dtype)


def rmat_edges(
    num_nodes: int,
    first_edge: int,
    num_edges: int,
    seed: int = 0,
    a: float = 0.57,
    b: float = 0.19,
    c: float = 0.19,
    device="cpu",
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Directed R-MAT edges number ``first_edge .. first_edge+num_edges-1``.

    Node ids are drawn in a ``2**ceil(log2 N)`` square and folded into
    ``[0, N)`` with a modulo.
    """
    levels = max(1, (num_nodes - 1).bit_length())
    t1 = int(a * 65536)
    t2 = int((a + b) * 65536)
    t3 = int((a + b + c) * 65536)
    idx = torch.arange(first_edge, first_edge + num_edges, dtype=torch.int64, device=device)
    row = torch.zeros_like(idx)
    col = torch.zeros_like(idx)
    bits = None
    for lvl in range(levels):
        if lvl % 4 == 0:
            bits = hash_stream(seed, 1000 + lvl // 4, idx)
        u = _lsr(bits, 16 * (lvl % 4)) & 0xFFFF
        # quadrant 0:(0,0) 1:(0,1) 2:(1,0) 3:(1,1)
        right = ((u >= t1) & (u < t2)) | (u >= t3)
        down = u >= t2
        row = (row << 1) | down.to(torch.int64)
        col = (col << 1) | right.to(torch.int64)
    return row % num_nodes, col % num_nodes


def uniform_edges(num_nodes: int, first_edge: int, num_edges: int, seed: int = 0, device="cpu"):
    idx = torch.arange(first_edge, first_edge + num_edges, dtype=torch.int64, device=device)
    row = (hash_stream(seed, 2000, idx) & _MASK63) % num_nodes
    col = (hash_stream(seed, 2001, idx) & _MASK63) % num_nodes
    return row, col


def undirected_unique_keys(
    num_nodes: int,
    num_undirected_edges: int,
    seed: int = 0,
    kind: str = "rmat",
    device="cpu",
    chunk: int = 1 << 24,
    oversample: float = 1.0,
    **rmat_kw,
) -> torch.Tensor:
    """Sorted unique keys ``lo * N + hi`` (lo < hi) of about the requested count.

    Edges are generated in chunks until enough distinct non-loop pairs exist;
    if there are more than requested, a hash-selected subset is kept so the
    result does not depend on chunking.
    """
    gen = rmat_edges if kind == "rmat" else uniform_edges
    kw = rmat_kw if kind == "rmat" else {}
    keys = torch.empty(0, dtype=torch.int64, device=device)
    produced = 0
    want = int(num_undirected_edges)
    rounds = 0
    while keys.numel() < want and rounds < 256:
        missing = want - keys.numel()
        n = min(chunk, max(1024, int(missing * max(1.0, oversample) * 1.1)))
        r, c = gen(num_nodes, produced, n, seed=seed, device=device, **kw)
        produced += n
        lo, hi = torch.minimum(r, c), torch.maximum(r, c)
        keep = lo != hi
        new = (lo * num_nodes + hi)[keep]
        keys = torch.unique(torch.cat([keys, new]))
        rounds += 1
    if keys.numel() > want:
        h = _lsr(hash_stream(seed, 3000, keys), 1)
        thr = int((want / keys.numel()) * float(1 << 63))
        keys = keys[h < thr]
    return keys


def synthetic_graph(
    num_nodes: int,
    num_undirected_edges: int,
    num_features: int,
    num_classes: int,
    seed: int = 0,
    kind: str = "rmat",
    device="cpu",
    feature_dtype=torch.float32,
    with_masks: bool = True,
    **rmat_kw,
) -> Tuple[Data, int]:
    """Symmetric graph with self-loops and GCN normalisation, N(0,1) features, uniform labels.

    Returns ``(data, num_classes)`` in the processed-file layout (unpermuted):
    ``edge_index`` is sorted by (row, col), ``edge_weight`` holds
    ``D^-1/2 (A + I) D^-1/2``.
    """
    from .graph_ops import gcn_normalize, symmetrize_with_self_loops

    keys = undirected_unique_keys(
        num_nodes, num_undirected_edges, seed=seed, kind=kind, device=device, **rmat_kw
    )
    edge_index = symmetrize_with_self_loops(keys, num_nodes)
    del keys
    edge_weight = gcn_normalize(edge_index, num_nodes)
    x = synthetic_features(num_nodes, num_features, seed, device=device, dtype=feature_dtype)
    y = synthetic_labels(num_nodes, num_classes, seed, device=device)
    data = Data(x=x, y=y, edge_index=edge_index, edge_weight=edge_weight)
    data.symmetric = True
    if with_masks:
        u = uniform01(seed, 4000, torch.arange(num_nodes, dtype=torch.int64, device=device))
        data.train_mask = u < 0.5
        data.val_mask = (u >= 0.5) & (u < 0.75)
        data.test_mask = u >= 0.75
    return data, num_classes


def synthetic_features(
    num_nodes: int,
    num_features: int,
    seed: int = 0,
    device="cpu",
    dtype=torch.float32,
    row_start: int = 0,
    row_stop: Optional[int] = None,
    chunk_rows: int = 1 << 20,
) -> torch.Tensor:
    """Rows ``[row_start, row_stop)`` of the N(0,1) feature matrix."""
    row_stop = num_nodes if row_stop is None else row_stop
    out = torch.empty((row_stop - row_start, num_features), dtype=dtype, device=device)
    for r0 in range(row_start, row_stop, chunk_rows):
        r1 = min(row_stop, r0 + chunk_rows)
        idx = torch.arange(r0 * num_features, r1 * num_features, dtype=torch.int64, device=device)
        out[r0 - row_start : r1 - row_start] = normal01(seed, 5000, idx, dtype).view(
            r1 - r0, num_features
        )
    return out


def synthetic_labels(num_nodes: int, num_classes: int, seed: int = 0, device="cpu") -> torch.Tensor:
    idx = torch.arange(num_nodes, dtype=torch.int64, device=device)
    return (hash_stream(seed, 6000, idx) & _MASK63) % num_classes
