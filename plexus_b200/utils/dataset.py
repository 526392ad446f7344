"""Offline graph preprocessing, format converters and the static 2-D partitioner.

Reference: plexus/utils/dataset.py — ``preprocess_graph`` (:29-249),
``write_to_mtx`` / ``mtx_to_pyg`` / ``tsv_to_pyg`` / ``print_nnz_stats``
(:252-367) and ``partition_graph_2d`` (:370-566).  File layouts are kept:

* ``processed_<name>.pt`` = ``torch.save((data, num_classes))``;
* partition directory: ``metadata.pt``, ``edge_index/{0,1}/{i}_{j}.pt``
  (global ids + weights), ``input_features/{i}_{j}.pt``,
  ``output_labels/{0,1}/{i}.pt``.

Besides the named datasets (which need PyTorch Geometric / OGB and are
imported lazily) the seeded synthetic kinds ``rmat`` and ``uniform`` are
accepted.
"""

from __future__ import annotations

import os
import re
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

import numpy as np
import torch

from ..data import graph_ops
from ..data.container import Data, load_processed, save_processed
from ..data.synthetic import synthetic_graph
from ..parallel.sharding import pad_dimension

NAMED_DATASETS = ("reddit", "products", "papers", "europe_osm", "protein", "amazon")
SYNTHETIC_DATASETS = ("rmat", "uniform")


def _row_normalize(x: torch.Tensor) -> torch.Tensor:
    """Scale every feature row to sum 1 (PyG ``NormalizeFeatures``)."""
    s = x.sum(dim=1, keepdim=True).clamp(min=1.0)
    return x / s


def _load_named(name: str, input_dir: str):
    """Raw ``(data, num_classes or None, unsupervised, directed)`` for a named dataset."""
    try:
        import torch_geometric.transforms as T  # noqa: F401
        from torch_geometric.datasets import Reddit, SuiteSparseMatrixCollection
    except Exception as e:  # pragma: no cover - optional dependency
        raise ImportError(
            f"dataset '{name}' needs torch_geometric (and ogb for products/papers); "
            "use name='rmat' or 'uniform' for a synthetic graph"
        ) from e
    if name == "reddit":
        ds = Reddit(root=input_dir)
        return ds[0], ds.num_classes, False, False
    if name in ("products", "papers"):
        from ogb.nodeproppred import PygNodePropPredDataset

        ds = PygNodePropPredDataset(
            name="ogbn-products" if name == "products" else "ogbn-papers100M", root=input_dir
        )
        return ds[0], ds.num_classes, False, name == "papers"
    if name == "europe_osm":
        ds = SuiteSparseMatrixCollection(input_dir, "DIMACS10", name)
        return ds[0], None, True, False
    # protein / amazon: input_dir is the path of a .pt file holding a Data object
    return torch.load(input_dir, weights_only=False), None, True, False


def degree_quantile_labels(edge_index: torch.Tensor, num_nodes: int, num_classes: int) -> torch.Tensor:
    """Label = index of the node's degree quantile bucket (for unlabeled graphs)."""
    deg = torch.bincount(edge_index[0], minlength=num_nodes).cpu().numpy()
    order = np.argsort(deg, kind="stable")
    y = np.zeros(num_nodes, dtype=np.int64)
    for i, bucket in enumerate(np.array_split(order, num_classes)):
        y[bucket] = i
    return torch.from_numpy(y)


def preprocess_data(
    data,
    num_classes: int,
    double_perm: bool = True,
    directed: bool = False,
    normalized: bool = False,
    seed: Optional[int] = None,
):
    """Normalise (unless already done), permute and return a processed ``Data``.

    With the double permutation two adjacency versions are stored,
    ``A1 = P A P2^T`` (even layers) and ``A2 = P2 A P^T`` (odd layers); the
    features follow the column permutation of ``A1``; ``y`` follows ``P`` and
    ``y_2`` follows ``P2``.
    """
    N = int(data.x.shape[0])
    dev = data.edge_index.device
    ei, ew = data.edge_index, getattr(data, "edge_weight", None)
    if not normalized:
        ei, ew = graph_ops.add_remaining_self_loops(ei, ew, N)
        ew = graph_ops.gcn_normalize(ei, N, ew)
    if directed:
        ei = torch.stack([ei[1], ei[0]])
    y = data.y.reshape(-1)
    if y.is_floating_point():
        y = torch.nan_to_num(y, nan=-1)
    y = y.to(torch.int64)

    gen = torch.Generator(device="cpu")
    gen.manual_seed(torch.initial_seed() if seed is None else seed)
    perm = torch.randperm(N, generator=gen).to(dev)
    perm2 = torch.randperm(N, generator=gen).to(dev) if double_perm else None

    out = Data()
    if double_perm:
        out.edge_index, out.edge_weight = graph_ops.permute_edges(ei, perm, perm2, ew)
        out.edge_index_2, out.edge_weight_2 = graph_ops.permute_edges(ei, perm2, perm, ew)
        out.x = data.x[perm2]
        out.y = y[perm]
        out.y_2 = y[perm2]
    else:
        out.edge_index, out.edge_weight = graph_ops.permute_edges(ei, perm, perm, ew)
        out.x = data.x[perm]
        out.y = y[perm]
    out.symmetric = bool(getattr(data, "symmetric", False)) and not directed
    for m in ("train_mask", "val_mask", "test_mask"):
        if hasattr(data, m) and getattr(data, m) is not None:
            setattr(out, m, getattr(data, m)[perm])
            if double_perm:
                setattr(out, m + "_2", getattr(data, m)[perm2])
    return out, num_classes


def preprocess_graph(
    name: str,
    input_dir: Optional[str],
    output_dir: str,
    double_perm: Optional[bool] = True,
    unsupervised: Optional[bool] = False,
    num_features: Optional[int] = 128,
    num_classes: Optional[int] = 32,
    directed: Optional[bool] = False,
    *,
    num_nodes: Optional[int] = None,
    num_edges: Optional[int] = None,
    seed: int = 0,
    device: str = "cpu",
) -> str:
    """Preprocess a dataset and save ``processed_<name>.pt`` in ``output_dir``.

    For ``name`` in ``rmat`` / ``uniform`` a synthetic graph of ``num_nodes``
    nodes and ``num_edges`` undirected edges is generated from ``seed``.
    """
    normalized = False
    if name in SYNTHETIC_DATASETS:
        if num_nodes is None or num_edges is None:
            raise ValueError("synthetic graphs need num_nodes and num_edges")
        data, num_classes = synthetic_graph(
            num_nodes, num_edges, num_features, num_classes, seed=seed, kind=name, device=device
        )
        normalized = True
    elif name in NAMED_DATASETS:
        data, nc, force_unsup, force_directed = _load_named(name, input_dir)
        unsupervised = unsupervised or force_unsup
        directed = directed or force_directed
        if not unsupervised:
            num_classes = nc
            data.x = _row_normalize(data.x)
    else:
        raise Exception(name + " dataset not supported")
    print("Read the original dataset.\n")

    if unsupervised and name not in SYNTHETIC_DATASETS:
        N = data.num_nodes
        data.x = _row_normalize(torch.rand(N, num_features))
        ei, ew = graph_ops.add_remaining_self_loops(data.edge_index, getattr(data, "edge_weight", None), N)
        data.edge_index, data.edge_weight = ei, graph_ops.gcn_normalize(ei, N, ew)
        normalized = True
        data.y = degree_quantile_labels(data.edge_index, N, num_classes)

    out, num_classes = preprocess_data(
        data, num_classes, double_perm=bool(double_perm), directed=bool(directed),
        normalized=normalized, seed=seed,
    )
    print("Normalized and permuted the graph.\n")
    out = out.to("cpu")
    os.makedirs(output_dir, exist_ok=True)
    path = os.path.join(output_dir, "processed_" + name + ".pt")
    save_processed(out, num_classes, path)
    print("Saved the preprocessed dataset to " + path)
    return path


# --------------------------------------------------------------------------
# converters and statistics
# --------------------------------------------------------------------------
def write_to_mtx(file_path: str, output_dir: str) -> str:
    """Write the (weighted) adjacency of a processed ``.pt`` file as MatrixMarket."""
    import scipy.sparse as sp
    from scipy.io import mmwrite

    data, _ = load_processed(file_path)
    n = int(data.x.shape[0])
    m = sp.coo_matrix(
        (data.edge_weight.cpu().numpy(), (data.edge_index[0].cpu().numpy(), data.edge_index[1].cpu().numpy())),
        shape=(n, n),
    )
    name = re.search(r"([^/]+)\.pt$", file_path).group(1)
    out = os.path.join(output_dir, name + ".mtx")
    mmwrite(out, m)
    print("Saved weighted graph adjacency matrix to " + out)
    return out


def mtx_to_pyg(mtx_file: str, output_file: str) -> None:
    """MatrixMarket pattern -> ``Data(edge_index, unit edge_weight, num_nodes)``."""
    from scipy.io import mmread

    m = mmread(mtx_file)
    r, c = m.nonzero()
    ei = torch.from_numpy(np.vstack((r, c))).long()
    d = Data(edge_index=ei, edge_weight=torch.ones(ei.shape[1]))
    d.num_nodes = m.shape[0]
    torch.save(d, output_file)
    print(f"Saved processed graph to {output_file}")


def tsv_to_pyg(tsv_file: str, output_file: str, N: int) -> None:
    """``src<TAB>dst<TAB>value`` lines -> ``Data(edge_index, edge_attr, num_nodes=N)``."""
    arr = np.loadtxt(tsv_file, delimiter="\t", ndmin=2)
    ei = torch.from_numpy(arr[:, :2].astype(np.int64)).t().contiguous()
    d = Data(edge_index=ei, edge_attr=torch.from_numpy(arr[:, 2].astype(np.float32)))
    d.num_nodes = N
    torch.save(d, output_file)


def print_nnz_stats(file_path: str, num_partitions: int):
    """Print the nnz of every 2-D block and balance statistics; returns the count matrix."""
    data, _ = load_processed(file_path)
    counts = graph_ops.block_nnz_counts(data.edge_index, data.num_nodes, num_partitions).float()
    for i in range(num_partitions):
        for j in range(num_partitions):
            print(f"row_partition_num: {i}, col_partition_num: {j}\n{counts[i, j]}\n")
    mn, mean, med, mx = counts.min().item(), counts.mean().item(), counts.median().item(), counts.max().item()
    print(f"Min: {mn}, Mean: {mean}, Median: {med}, Max: {mx}")
    print(f"Max/Mean: {mx / mean}, Max/Min: {mx / mn if mn else float('inf')}")
    return counts


# --------------------------------------------------------------------------
# static 2-D partitioner
# --------------------------------------------------------------------------
def _atomic_save(obj, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _bucket_edges(edge_index, edge_weight, chunk: int, p: int):
    """Group edges by block with one sort; returns (edge_index, weight, offsets[p*p+1])."""
    bi = torch.div(edge_index[0], chunk, rounding_mode="floor")
    bj = torch.div(edge_index[1], chunk, rounding_mode="floor")
    bid = bi * p + bj
    order = torch.argsort(bid, stable=True)
    counts = torch.bincount(bid, minlength=p * p)
    offs = torch.zeros(p * p + 1, dtype=torch.int64)
    offs[1:] = torch.cumsum(counts, 0)
    return edge_index[:, order], edge_weight[order], offs


def partition_graph_2d(file_path: str, num_partitions: int, output_dir: str) -> None:
    """Split a processed graph into ``p x p`` files for parallel loading.

    Edges are bucketed by block with a single sort instead of one mask over
    the whole edge list per block.
    """
    data, num_classes = load_processed(file_path)
    p = int(num_partitions)
    double_perm = hasattr(data, "edge_index_2")
    N, F = int(data.x.shape[0]), int(data.x.shape[1])
    chunk_n = pad_dimension(N, p) // p
    chunk_f = pad_dimension(F, p) // p

    os.makedirs(output_dir, exist_ok=True)
    _atomic_save((N, F, num_classes), os.path.join(output_dir, "metadata.pt"))
    for sub in ["edge_index/0", "input_features", "output_labels/0"] + (
        ["edge_index/1", "output_labels/1"] if double_perm else []
    ):
        os.makedirs(os.path.join(output_dir, sub), exist_ok=True)

    versions = [(data.edge_index.cpu(), data.edge_weight.cpu())]
    if double_perm:
        versions.append((data.edge_index_2.cpu(), data.edge_weight_2.cpu()))
    bucketed = [_bucket_edges(ei, ew, chunk_n, p) for ei, ew in versions]
    labels = [data.y.cpu()] + ([data.y_2.cpu()] if double_perm else [])
    x = data.x.cpu()

    def write_block(i: int, j: int) -> None:
        for v, (ei, ew, offs) in enumerate(bucketed):
            a, b = int(offs[i * p + j]), int(offs[i * p + j + 1])
            _atomic_save(
                (ei[:, a:b].clone(), ew[a:b].clone()),
                os.path.join(output_dir, "edge_index", str(v), f"{i}_{j}.pt"),
            )
        r0, r1 = i * chunk_n, min((i + 1) * chunk_n, N)
        f0, f1 = j * chunk_f, min((j + 1) * chunk_f, F)
        _atomic_save(x[r0:r1, f0:f1].clone(), os.path.join(output_dir, "input_features", f"{i}_{j}.pt"))
        if j == 0:
            for v, y in enumerate(labels):
                _atomic_save(y[r0:r1].clone(), os.path.join(output_dir, "output_labels", str(v), f"{i}.pt"))

    with ThreadPoolExecutor(max_workers=min(os.cpu_count() or 1, p * p)) as pool:
        futures = [pool.submit(write_block, i, j) for i in range(p) for j in range(p)]
        for f in futures:
            f.result()
    extra = {"symmetric": bool(getattr(data, "symmetric", False))}
    _atomic_save(extra, os.path.join(output_dir, "extra.pt"))
