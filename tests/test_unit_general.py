import pytest
import torch

from plexus_b200.parallel import grid as G
from plexus_b200.parallel.sharding import (
    block_range, depth_slice, extract_local_params_from_full_params, pad_dimension, padded_channels, shard_2d,
)


def test_pad_dimension():
    assert pad_dimension(10, 4) == 12
    assert pad_dimension(12, 4) == 12
    assert pad_dimension(10, 2, 3) == 12
    assert pad_dimension(13, 2, 3) == 18
    assert pad_dimension(0, 4) == 0
    assert pad_dimension(7, 1) == 7


def test_padded_channels():
    assert padded_channels(100, 2, 2, 8) == 112  # multiple of 2*lcm(2,8)=16
    assert padded_channels(100, 2, 1, 1) == 100
    assert padded_channels(47, 8, 1, 8) == 64
    assert padded_channels(47, 2, 4, 1) == 48


@pytest.mark.parametrize("shape", [(1, 1, 1), (2, 1, 1), (1, 2, 1), (2, 2, 2), (4, 2, 1), (2, 4, 8)])
def test_rank_coords_roundtrip(shape):
    X, Y, Z = shape
    seen = set()
    for r in range(X * Y * Z):
        x, y, z = G.coords_of(r, X, Y, Z)
        assert 0 <= x < X and 0 <= y < Y and 0 <= z < Z
        assert G.rank_of(x, y, z, X, Y, Z) == r
        assert r == z * X * Y + x * Y + y  # Y fastest, then X, then Z
        seen.add((x, y, z))
    assert len(seen) == X * Y * Z


def test_line_ranks():
    X, Y, Z = 2, 2, 2
    assert G.line_ranks("y", 0, 0, 0, X, Y, Z) == [0, 1]
    assert G.line_ranks("x", 0, 0, 0, X, Y, Z) == [0, 2]
    assert G.line_ranks("z", 0, 0, 0, X, Y, Z) == [0, 4]
    assert G.line_ranks("x", 1, 1, 1, X, Y, Z) == [5, 7]
    with pytest.raises(ValueError):
        G.line_ranks("w", 0, 0, 0, X, Y, Z)


def test_axis_role_rotation():
    assert G.axis_roles(0) == ("x", "y", "z")
    assert G.axis_roles(1) == ("z", "x", "y")
    assert G.axis_roles(2) == ("y", "z", "x")
    assert G.axis_roles(3) == ("x", "y", "z")
    # output layout of layer l (rows by depth, cols by outer) == input layout of l+1 (rows by outer, cols by inner)
    for l in range(6):
        o, i, d = G.axis_roles(l)
        o2, i2, d2 = G.axis_roles(l + 1)
        assert o2 == d and i2 == o and d2 == i


def test_loss_axes():
    assert G.loss_axes(1) == ("z", "x")
    assert G.loss_axes(2) == ("y", "z")
    assert G.loss_axes(3) == ("x", "y")
    assert G.loss_axes(4) == ("z", "x")


def test_grid_info_single_process():
    g = G.ProcessGrid.build(1, 1, 1)
    sizes, ranks, groups = g.info(("z", "x", "y"))
    assert sizes == [1, 1, 1] and ranks == [0, 0, 0] and groups == [None, None, None]
    with pytest.raises(AssertionError):
        g.info(("x", "x"))
    with pytest.raises(ValueError):
        g.info(("q",))
    with pytest.raises(ValueError):
        G.ProcessGrid.build(2, 1, 1, rank=0, world_size=1)


def test_comm_handle_names():
    g = G.ProcessGrid(X=2, Y=3, Z=4, rank=2 * 6 + 1 * 3 + 2, world_size=24)
    h = G.CommHandle(g)
    assert (h.G_intra_r, h.G_intra_c, h.G_intra_d) == (2, 3, 4)
    assert h.intra_layer_row_parallel_rank == 1
    assert h.intra_layer_column_parallel_rank == 2
    assert h.intra_layer_depth_parallel_rank == 2


def test_shard_2d_matches_dense_slicing():
    full = torch.arange(7 * 5, dtype=torch.float32).view(7, 5)
    padded = torch.zeros(8, 6)
    padded[:7, :5] = full
    for ri in range(4):
        for ci in range(3):
            blk = shard_2d(full, 4, ri, 3, ci)
            assert torch.equal(blk, padded[ri * 2:(ri + 1) * 2, ci * 2:(ci + 1) * 2])


def test_block_range_and_depth_slice():
    assert block_range(10, 4, 0) == (0, 3)
    assert block_range(10, 4, 3) == (9, 12)
    t = torch.arange(12)
    assert torch.equal(depth_slice(t, 3, 1), torch.arange(4, 8))
    with pytest.raises(ValueError):
        depth_slice(torch.arange(10), 3, 0)


def test_extract_local_params_single_rank():
    w = torch.randn(6, 4)
    flat = extract_local_params_from_full_params(w, None, None, None)
    assert torch.equal(flat, w.reshape(-1))


def test_weight_shard_init_equals_slices_of_the_full_matrix():
    """Every (row block, column block, depth slice) generated on its own equals the slice of the
    zero-padded full matrix; values do not depend on how the matrix is cut."""
    import torch
    from plexus_b200.models.gcn_conv import init_full_weight, init_weight_shard

    in_ch, out_ch, layer, seed = 100, 47, 2, 11
    full = init_full_weight(in_ch, out_ch, layer, seed)
    assert full.shape == (in_ch, out_ch)
    bound = 1.0 / in_ch ** 0.5
    assert full.abs().max() <= bound and full.std() > 0.4 * bound
    assert not torch.equal(full, init_full_weight(in_ch, out_ch, layer + 1, seed))
    for inner, outer, depth in [(1, 1, 1), (2, 2, 2), (4, 1, 2), (1, 8, 1)]:
        pin = -(-in_ch // (inner * depth * 8)) * inner * depth * 8
        pout = -(-out_ch // (outer * 8)) * outer * 8
        padded = torch.nn.functional.pad(full, (0, pout - out_ch, 0, pin - in_ch))
        lr, lc = pin // inner, pout // outer
        for i in range(inner):
            for o in range(outer):
                block = padded[i * lr:(i + 1) * lr, o * lc:(o + 1) * lc].reshape(-1)
                per = block.numel() // depth
                for d in range(depth):
                    got = init_weight_shard(in_ch, out_ch, layer, seed, i * lr, o * lc, lc, d * per, per, "cpu")
                    assert torch.equal(got, block[d * per:(d + 1) * per]), (inner, outer, depth, i, o, d)


def test_two_shot_row_segments_cover_the_rows_exactly_once():
    from types import SimpleNamespace

    from plexus_b200.parallel.fused import _segment

    for p in (2, 3, 4, 8):
        for rows in (0, 1, 5, 7, 8, 1003, 4096):
            seg, ranges = _segment(SimpleNamespace(p=p), rows)
            assert seg * p >= rows and len(ranges) == p
            covered = []
            for q, (r0, n) in enumerate(ranges):
                assert 0 <= n <= seg and r0 == min(q * seg, rows)
                covered += list(range(r0, r0 + n))
            assert covered == list(range(rows)), (p, rows)


def test_emulator_and_extension_expose_the_same_peer_memory_api():
    """Every kernel entry point the fused collectives call exists in the emulation, and (when the
    extension is built) in the extension under the same name."""
    import os
    import re

    from plexus_b200.ops import _ext
    from plexus_b200.parallel import emulator

    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    names = set()
    for f in ("fused.py", "symm.py"):
        src = open(os.path.join(here, "plexus_b200", "parallel", f)).read()
        names |= set(re.findall(r"\b(?:C|_Backend\.load\(\)|_C\(\))\.([a-z_0-9]+)\(", src))
    assert {"symm_alloc", "symm_open", "push_copy", "reduce_slots", "reduce_segment", "gather_segments"} <= names
    for n in sorted(names):
        assert hasattr(emulator.C, n), f"emulator lacks {n}"
    if _ext.available():
        try:
            ext = _ext.load()
        except (ImportError, OSError):  # no CUDA runtime libraries on this machine
            return
        for n in sorted(names):
            assert hasattr(ext, n), f"extension lacks {n}"
