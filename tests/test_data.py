"""Synthetic graphs, preprocessing, partition files and the per-rank loader (CPU)."""

import os

import pytest
import torch

from helpers import dense_adj, small_processed_graph


def test_rmat_is_deterministic_and_chunk_independent():
    from plexus_b200.data.synthetic import rmat_edges, synthetic_graph

    r1, c1 = rmat_edges(1000, 0, 5000, seed=3)
    r2, c2 = rmat_edges(1000, 0, 5000, seed=3)
    assert torch.equal(r1, r2) and torch.equal(c1, c2)
    # any sub-range of edge indices can be generated on its own
    ra, ca = rmat_edges(1000, 1234, 100, seed=3)
    assert torch.equal(ra, r1[1234:1334]) and torch.equal(ca, c1[1234:1334])
    r3, _ = rmat_edges(1000, 0, 5000, seed=4)
    assert not torch.equal(r1, r3)
    d1, _ = synthetic_graph(500, 3000, 8, 4, seed=1)
    d2, _ = synthetic_graph(500, 3000, 8, 4, seed=1)
    assert torch.equal(d1.edge_index, d2.edge_index) and torch.equal(d1.x, d2.x) and torch.equal(d1.y, d2.y)


def test_rmat_is_skewed_and_edge_count_close_to_request():
    from plexus_b200.data.synthetic import synthetic_graph

    n, e = 4096, 40000
    d, _ = synthetic_graph(n, e, 4, 3, seed=0)
    nnz = d.edge_index.shape[1]
    assert abs(nnz - (2 * e + n)) < 0.05 * (2 * e + n)
    deg = torch.bincount(d.edge_index[0], minlength=n)
    assert deg.max() > 8 * deg.float().mean()  # power-law tail
    assert deg.min() >= 1  # self loops


def test_normalisation_is_symmetric_gcn_norm():
    from plexus_b200.data.synthetic import synthetic_graph

    n = 300
    d, _ = synthetic_graph(n, 1500, 4, 3, seed=2, kind="uniform")
    A = dense_adj(d.edge_index, d.edge_weight, n)
    pattern = (A != 0).double()
    assert torch.equal(pattern, pattern.t())
    assert torch.all(torch.diag(pattern) == 1)
    deg = pattern.sum(1)
    want = pattern / torch.sqrt(deg).unsqueeze(1) / torch.sqrt(deg).unsqueeze(0)
    assert torch.allclose(A, want, atol=1e-6)


def test_double_permutation_equals_matrix_products():
    from plexus_b200.data import graph_ops

    n = 40
    g = torch.Generator().manual_seed(0)
    ei = torch.randint(0, n, (2, 200), generator=g)
    ei = torch.unique(ei, dim=1)
    ew = torch.rand(ei.shape[1], generator=g)
    A = dense_adj(ei, ew, n)
    perm, perm2 = torch.randperm(n, generator=g), torch.randperm(n, generator=g)
    P = torch.zeros(n, n, dtype=torch.float64)
    P[torch.arange(n), perm] = 1
    P2 = torch.zeros(n, n, dtype=torch.float64)
    P2[torch.arange(n), perm2] = 1
    e1, w1 = graph_ops.permute_edges(ei, perm, perm2, ew)
    e2, w2 = graph_ops.permute_edges(ei, perm2, perm, ew)
    assert torch.allclose(dense_adj(e1, w1, n), P @ A @ P2.t())
    assert torch.allclose(dense_adj(e2, w2, n), P2 @ A @ P.t())
    # sorted by (row, col)
    key = e1[0] * n + e1[1]
    assert torch.all(key[1:] > key[:-1])


def test_coo_to_csr_and_transpose():
    from plexus_b200.data import graph_ops

    g = torch.Generator().manual_seed(1)
    rows, cols = 17, 23
    ei = torch.unique(torch.stack([torch.randint(0, rows, (90,), generator=g),
                                   torch.randint(0, cols, (90,), generator=g)]), dim=1)
    ew = torch.rand(ei.shape[1], generator=g)
    order = torch.randperm(ei.shape[1], generator=g)
    crow, col, val = graph_ops.coo_to_csr(ei[0][order], ei[1][order], ew[order], rows, cols)
    A = graph_ops.csr_tensor(crow, col, val, (rows, cols))
    dense = torch.zeros(rows, cols)
    dense[ei[0], ei[1]] = ew
    assert torch.allclose(A.to_dense(), dense)
    assert crow.dtype == torch.int32 and col.dtype == torch.int32
    At = graph_ops.csr_transpose(A)
    assert torch.allclose(At.to_dense(), dense.t())


def _loader_outputs(grid_shape, rank, data, nc, layers, data_dir=None):
    from plexus_b200 import runtime
    from plexus_b200.parallel import grid as G
    from plexus_b200.utils.dataloader import DataLoader

    X, Y, Z = grid_shape
    G.set_grid(G.ProcessGrid(X=X, Y=Y, Z=Z, rank=rank, world_size=X * Y * Z))
    runtime.flags.dtype, runtime.flags.channel_align = torch.float32, 1
    if data_dir is None:
        return DataLoader(None, layers, data=(data, nc), device=torch.device("cpu")).load()
    return DataLoader(data_dir, layers, device=torch.device("cpu")).load()


@pytest.mark.parametrize("grid_shape", [(2, 1, 1), (1, 2, 2), (2, 2, 2), (4, 2, 1)])
@pytest.mark.parametrize("double_perm", [True, False])
def test_loader_shards_match_dense_slicing(grid_shape, double_perm):
    from plexus_b200.parallel import grid as G
    from plexus_b200.parallel.sharding import pad_dimension

    n, f, layers = 53, 7, 4
    data, nc = small_processed_graph(n=n, e=200, f=f, c=5, seed=4, double_perm=double_perm)
    X, Y, Z = grid_shape
    dense = [dense_adj(data.edge_index, data.edge_weight, n)]
    if double_perm:
        dense.append(dense_adj(data.edge_index_2, data.edge_weight_2, n))
    for rank in range(X * Y * Z):
        adj, feats, labels, N, F, C = _loader_outputs(grid_shape, rank, data, nc, layers)
        x, y, z = G.coords_of(rank, X, Y, Z)
        sizes, coords = {"x": X, "y": Y, "z": Z}, {"x": x, "y": y, "z": z}
        assert len(adj) == (4 if double_perm else 3)
        for i, (A, At) in enumerate(adj):
            outer, _inner, depth = G.axis_roles(i)
            rs, cs = pad_dimension(n, sizes[depth]) // sizes[depth], pad_dimension(n, sizes[outer]) // sizes[outer]
            full = torch.zeros(rs * sizes[depth], cs * sizes[outer], dtype=torch.float64)
            full[:n, :n] = dense[i % 2 if double_perm else 0]
            want = full[coords[depth] * rs:(coords[depth] + 1) * rs, coords[outer] * cs:(coords[outer] + 1) * cs]
            assert torch.allclose(A.to_dense().double(), want, atol=1e-7), (rank, i)
            assert torch.allclose(At.to_dense().double(), want.t(), atol=1e-7), (rank, i, "T")
        # features: rows over X, columns over Y (padded to Y*Z), flat slice over Z
        rows = pad_dimension(n, X) // X
        fpad = pad_dimension(f, Y, Z)
        xfull = torch.zeros(rows * X, fpad)
        xfull[:n, :f] = data.x
        blk = xfull[x * rows:(x + 1) * rows, y * (fpad // Y):(y + 1) * (fpad // Y)].reshape(-1)
        step = blk.numel() // Z
        assert torch.allclose(feats.detach(), blk[z * step:(z + 1) * step])
        assert feats.requires_grad
        # labels: rows over the depth axis of the last layer, padding rows are -1
        row_axis, _ = G.loss_axes(layers)
        ls = pad_dimension(n, sizes[row_axis]) // sizes[row_axis]
        ysrc = data.y_2 if (double_perm and layers % 2 == 0) else data.y
        yfull = torch.full((ls * sizes[row_axis],), -1, dtype=torch.int64)
        yfull[:n] = ysrc
        assert torch.equal(labels, yfull[coords[row_axis] * ls:(coords[row_axis] + 1) * ls])


@pytest.mark.parametrize("double_perm", [True, False])
def test_partition_files_round_trip(tmp_path, double_perm):
    from plexus_b200.data.container import save_processed
    from plexus_b200.utils.dataset import partition_graph_2d

    n, f, layers = 61, 9, 3
    data, nc = small_processed_graph(n=n, e=260, f=f, c=4, seed=6, double_perm=double_perm)
    single = tmp_path / "single"
    parts = tmp_path / "parts"
    single.mkdir()
    parts.mkdir()
    save_processed(data, nc, str(single / "processed_rmat.pt"))
    partition_graph_2d(str(single / "processed_rmat.pt"), 3, str(parts))
    assert (parts / "metadata.pt").exists() and (parts / "edge_index" / "0" / "2_1.pt").exists()
    assert (parts / "edge_index" / "1").exists() == double_perm
    for rank in range(4):
        a = _loader_outputs((2, 1, 2), rank, None, None, layers, data_dir=str(single))
        b = _loader_outputs((2, 1, 2), rank, None, None, layers, data_dir=str(parts))
        assert a[3:] == b[3:]
        for (A1, T1), (A2, T2) in zip(a[0], b[0]):
            assert torch.allclose(A1.to_dense(), A2.to_dense()) and torch.allclose(T1.to_dense(), T2.to_dense())
        assert torch.allclose(a[1].detach(), b[1].detach()) and torch.equal(a[2], b[2])


def test_missing_or_corrupt_partition_file_is_reported(tmp_path):
    from plexus_b200.data.container import save_processed
    from plexus_b200.utils.dataset import partition_graph_2d

    data, nc = small_processed_graph(n=40, e=150, f=4, c=3, seed=1)
    save_processed(data, nc, str(tmp_path / "processed_rmat.pt"))
    parts = tmp_path / "parts"
    parts.mkdir()
    partition_graph_2d(str(tmp_path / "processed_rmat.pt"), 2, str(parts))
    victim = parts / "edge_index" / "0" / "0_0.pt"
    victim.write_bytes(victim.read_bytes()[:20])  # truncated
    with pytest.raises(RuntimeError, match="corrupt partition file"):
        _loader_outputs((1, 1, 1), 0, None, None, 2, data_dir=str(parts))
    os.remove(victim)
    with pytest.raises(FileNotFoundError):
        _loader_outputs((1, 1, 1), 0, None, None, 2, data_dir=str(parts))


def test_preprocess_graph_synthetic_and_converters(tmp_path):
    from plexus_b200.data.container import load_processed
    from plexus_b200.utils import dataset as ds

    path = ds.preprocess_graph("rmat", None, str(tmp_path), num_features=6, num_classes=3,
                               num_nodes=200, num_edges=900, seed=5)
    data, nc = load_processed(path)
    assert nc == 3 and data.x.shape == (200, 6) and hasattr(data, "edge_index_2") and hasattr(data, "y_2")
    mtx = ds.write_to_mtx(path, str(tmp_path))
    ds.mtx_to_pyg(mtx, str(tmp_path / "back.pt"))
    back = torch.load(tmp_path / "back.pt", weights_only=False)
    assert back.edge_index.shape[1] == data.edge_index.shape[1] and back.num_nodes == 200
    counts = ds.print_nnz_stats(path, 2)
    assert int(counts.sum()) == data.edge_index.shape[1]
    tsv = tmp_path / "g.tsv"
    tsv.write_text("0\t1\t0.5\n1\t2\t1.5\n")
    ds.tsv_to_pyg(str(tsv), str(tmp_path / "t.pt"), 3)
    t = torch.load(tmp_path / "t.pt", weights_only=False)
    assert t.edge_index.tolist() == [[0, 1], [1, 2]] and t.num_nodes == 3
    with pytest.raises(Exception, match="not supported"):
        ds.preprocess_graph("nope", None, str(tmp_path))


def test_degree_quantile_labels():
    from plexus_b200.utils.dataset import degree_quantile_labels

    ei = torch.tensor([[0, 0, 0, 1, 1, 2], [1, 2, 3, 0, 2, 0]])
    y = degree_quantile_labels(ei, 4, 2)
    assert y.tolist() == [1, 1, 0, 0]


def test_named_dataset_branches_with_stand_in_dataset_packages(tmp_path, monkeypatch):
    """The named-dataset branch of ``preprocess_graph`` (reddit, ogbn-products, ogbn-papers100M,
    SuiteSparse europe_osm, a saved Data file) against stand-ins for torch_geometric / ogb: the real
    packages cannot be installed here, so small fakes with the same call surface take their place."""
    import sys
    import types

    from plexus_b200.data.container import Data
    from plexus_b200.utils import dataset as ds_mod

    def small_graph(n, e, f, classes, seed, with_xy=True):
        g = torch.Generator().manual_seed(seed)
        ei = torch.randint(0, n, (2, e), generator=g)
        d = Data(edge_index=ei, num_nodes=n)
        if with_xy:
            d.x = torch.rand(n, f, generator=g)
            d.y = torch.randint(0, classes, (n,), generator=g)
        return d

    calls = []

    class FakeSet:
        def __init__(self, data, num_classes):
            self._d, self.num_classes = data, num_classes

        def __getitem__(self, i):
            assert i == 0
            return self._d

    def Reddit(root):
        calls.append(("reddit", root))
        return FakeSet(small_graph(60, 300, 12, 7, 1), 7)

    def SuiteSparseMatrixCollection(root, group, name):
        calls.append(("suitesparse", root, group, name))
        return FakeSet(small_graph(50, 200, 0, 0, 2, with_xy=False), None)

    def PygNodePropPredDataset(name, root):
        calls.append(("ogb", name, root))
        d = small_graph(70, 350, 10, 5, 3)
        d.y = d.y.unsqueeze(1)  # ogb stores labels as a column
        return FakeSet(d, 5)

    tg = types.ModuleType("torch_geometric")
    tg_t = types.ModuleType("torch_geometric.transforms")
    tg_d = types.ModuleType("torch_geometric.datasets")
    tg_d.Reddit, tg_d.SuiteSparseMatrixCollection = Reddit, SuiteSparseMatrixCollection
    tg.transforms, tg.datasets = tg_t, tg_d
    ogb = types.ModuleType("ogb")
    ogb_n = types.ModuleType("ogb.nodeproppred")
    ogb_n.PygNodePropPredDataset = PygNodePropPredDataset
    ogb.nodeproppred = ogb_n
    for name, mod in (("torch_geometric", tg), ("torch_geometric.transforms", tg_t),
                      ("torch_geometric.datasets", tg_d), ("ogb", ogb), ("ogb.nodeproppred", ogb_n)):
        monkeypatch.setitem(sys.modules, name, mod)

    out = str(tmp_path / "out")
    # supervised sets keep their labels and class count; features are row-normalised
    for name, n, classes in (("reddit", 60, 7), ("products", 70, 5), ("papers", 70, 5)):
        path = ds_mod.preprocess_graph(name, str(tmp_path / "raw"), out, double_perm=True, seed=4)
        data, nc = ds_mod.load_processed(path)
        assert nc == classes and data.x.shape[0] == n
        assert torch.allclose(data.x.sum(dim=1), torch.ones(n), atol=1e-5)
        assert int(data.y.max()) < classes and data.edge_weight.numel() == data.edge_index.shape[1]
    raw = str(tmp_path / "raw")
    assert ("ogb", "ogbn-products", raw) in calls and ("ogb", "ogbn-papers100M", raw) in calls
    # unlabeled sets: random normalised features and degree-quantile labels with the requested sizes
    path = ds_mod.preprocess_graph("europe_osm", str(tmp_path / "raw"), out, num_features=9, num_classes=4, seed=4)
    data, nc = ds_mod.load_processed(path)
    assert nc == 4 and data.x.shape == (50, 9) and set(data.y.tolist()) == {0, 1, 2, 3}
    assert ("suitesparse", str(tmp_path / "raw"), "DIMACS10", "europe_osm") in calls
    saved = str(tmp_path / "protein.pt")
    torch.save(small_graph(40, 160, 0, 0, 5, with_xy=False), saved)
    path = ds_mod.preprocess_graph("protein", saved, out, num_features=6, num_classes=3, seed=4)
    data, nc = ds_mod.load_processed(path)
    assert nc == 3 and data.x.shape == (40, 6)
