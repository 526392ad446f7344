"""Rank-local generation of synthetic shards equals slicing the globally built graph."""

import pytest
import torch

from helpers import run_distributed

N, RAW, F, C, SEED = 301, 2400, 10, 7, 4


def _shards_equal(a, b):
    assert a.shape == b.shape
    assert torch.equal(a.crow_indices(), b.crow_indices())
    assert torch.equal(a.col_indices(), b.col_indices())
    assert torch.allclose(a.values(), b.values(), rtol=1e-6, atol=0)


def _compare(rank, world, grid, layers):
    import plexus_b200 as plx
    from plexus_b200.data.sharded_synthetic import ShardedSyntheticGraph, synthetic_graph_from_raw_edges
    from plexus_b200.utils.dataloader import DataLoader
    from plexus_b200.utils.dataset import preprocess_data

    plx.init(*grid, dtype=torch.float32)
    raw, nc = synthetic_graph_from_raw_edges(N, RAW, F, C, seed=SEED)
    data, _ = preprocess_data(raw, nc, double_perm=True, normalized=True, seed=SEED)
    ref = DataLoader(None, layers, data=(data, nc))
    adj_r, x_r, y_r, n_r, f_r, c_r = ref.load()

    src = ShardedSyntheticGraph(N, RAW, F, C, seed=SEED, chunk=500)  # several chunks and merges
    got = DataLoader(None, layers, source=src)
    adj_g, x_g, y_g, n_g, f_g, c_g = got.load()

    assert (n_g, f_g, c_g) == (n_r, f_r, c_r)
    assert src.nnz_total == data.edge_index.shape[1]
    assert len(adj_g) == len(adj_r)
    for (A, At), (B, Bt) in zip(adj_g, adj_r):
        _shards_equal(A, B)
        _shards_equal(At, Bt)
    assert torch.equal(x_g.detach(), x_r.detach())
    assert torch.equal(y_g, y_r)
    for m in ("train_mask", "val_mask", "test_mask"):
        assert torch.equal(got.masks[m], ref.masks[m]), m
    plx.shutdown()


@pytest.mark.parametrize("grid,layers", [((1, 1, 1), 3), ((2, 2, 1), 3), ((1, 2, 2), 2), ((2, 2, 2), 4)])
def test_sharded_generation_equals_global_pipeline(grid, layers):
    world = grid[0] * grid[1] * grid[2]
    run_distributed(_compare, world, grid, layers)


def test_degrees_do_not_depend_on_chunking_or_rank_count():
    from plexus_b200.data.sharded_synthetic import ShardedSyntheticGraph

    a = ShardedSyntheticGraph(N, RAW, F, C, seed=SEED, chunk=100).inverse_sqrt_degree()
    b = ShardedSyntheticGraph(N, RAW, F, C, seed=SEED, chunk=1 << 20).inverse_sqrt_degree()
    assert torch.equal(a, b)
    assert a.shape == (N,) and bool((a > 0).all()) and bool((a <= 1).all())


def _partition_worker(rank, world, outdir):
    import plexus_b200 as plx
    from plexus_b200.data.sharded_synthetic import ShardedSyntheticGraph, write_partition_tree
    from plexus_b200.utils.dataloader import DataLoader

    plx.init(2, 1, 2, dtype=torch.float32)
    src = ShardedSyntheticGraph(N, RAW, F, C, seed=SEED, chunk=700)
    write_partition_tree(src, 3, outdir, blocks_per_pass=2)   # 3 x 3 files, written by 4 ranks
    from_files = DataLoader(outdir, 3)
    adj_f, x_f, y_f, n_f, f_f, c_f = from_files.load()
    direct = DataLoader(None, 3, source=ShardedSyntheticGraph(N, RAW, F, C, seed=SEED))
    adj_d, x_d, y_d, n_d, f_d, c_d = direct.load()
    assert (n_f, f_f, c_f) == (n_d, f_d, c_d) and from_files.symmetric and from_files.double_perm
    for (A, At), (B, Bt) in zip(adj_f, adj_d):
        _shards_equal(A, B)
        _shards_equal(At, Bt)
    assert torch.equal(x_f.detach(), x_d.detach()) and torch.equal(y_f, y_d)
    plx.shutdown()


def test_partition_tree_written_from_the_generator_loads_like_the_direct_source(tmp_path):
    run_distributed(_partition_worker, 4, str(tmp_path / "parts"))
    import os

    assert os.path.exists(tmp_path / "parts" / "metadata.pt")
    assert len(os.listdir(tmp_path / "parts" / "edge_index" / "1")) == 9
