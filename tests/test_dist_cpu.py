"""3D-parallel GCN over gloo ranks on the CPU versus the serial dense oracle."""

import pytest
import torch

from helpers import oracle, run_distributed, small_processed_graph


def _worker(rank, world, grid, num_layers, double_perm, n, f, c, hidden, fuse, flags):
    import plexus_b200 as plx
    from plexus_b200.models.cross_entropy import parallel_cross_entropy
    from plexus_b200.models.net import Net
    from plexus_b200.utils.checkpoint import _cut_features, _cut_weight
    from plexus_b200.utils.dataloader import DataLoader

    torch.manual_seed(0)
    comm = None
    if flags.get("emulate_peer_memory"):
        # the fused collectives' host code against the shared-memory emulation of the kernels
        from plexus_b200.parallel import emulator, fused

        emulator.enable()
        comm = "fused"
        fused.SMALL_MESSAGE_BYTES = flags.get("small_bytes", fused.SMALL_MESSAGE_BYTES)
        fused.ONE_SHOT_MAX_RANKS = flags.get("one_shot_ranks", fused.ONE_SHOT_MAX_RANKS)
        fused.TWO_SHOT = flags.get("two_shot", False)
        fused.MAX_MESSAGE_BYTES = flags.get("max_message_bytes", fused.MAX_MESSAGE_BYTES)
        fused.ROW_BLOCK_MULTIPLE = flags.get("row_block_multiple", fused.ROW_BLOCK_MULTIPLE)
        fused.PIPELINE = flags.get("pipeline", False)
        fused.PIPELINE_MIN_BYTES = flags.get("pipeline_min_bytes", fused.PIPELINE_MIN_BYTES)
        fused.IN_KERNEL_REDUCE = flags.get("in_kernel", False)
        fused.SEGMENT_REDUCE = flags.get("segment_reduce", False)
        fused.XENT_EXCHANGE = flags.get("xent_exchange", False)
    plx.init(*grid, device="cpu", dtype=torch.float64, channel_align=flags.get("align", 1),
             block_aggregation=flags.get("block", False), overlap_aggregation=flags.get("overlap", False),
             tune_gemms=flags.get("tune", False), comm=comm)
    if flags.get("block"):
        from plexus_b200.models import gcn_conv
        gcn_conv.MAX_ROWS_PER_CHUNK = 17
    data, nc = small_processed_graph(n=n, e=4 * n, f=f, c=c, seed=5, double_perm=double_perm)
    loader = DataLoader(None, num_layers, data=(data, nc), dtype=torch.float64)
    adj, feats, labels, N, F, C = loader.load()
    model = Net(num_layers, F, hidden, C, fuse_layers=fuse, seed=11, order=flags.get("order", "auto")).double()
    out = model(feats, adj)
    loss = parallel_cross_entropy(out, labels, num_layers, N, C)
    loss.backward()

    ref_loss, ref_gw, ref_gx, _ = oracle(data, nc, num_layers, hidden, seed=11)
    assert torch.allclose(loss.detach(), ref_loss, rtol=1e-9, atol=1e-11), (loss.item(), ref_loss.item())
    for l, layer in enumerate(model.layers):
        want = _cut_weight(layer, ref_gw[l])
        got = layer.weight.grad
        assert got.shape == want.shape
        assert torch.allclose(got, want, rtol=1e-8, atol=1e-11), f"layer {l} weight grad"
    want_x = _cut_features(ref_gx, feats)
    assert torch.allclose(feats.grad, want_x, rtol=1e-8, atol=1e-11), "feature grad"
    if flags.get("emulate_peer_memory"):
        from plexus_b200.parallel import emulator

        from plexus_b200.parallel import fused

        emulator.ops.check_status()
        assert emulator.ops.launch_count > 0  # the emulated kernels really carried the collectives
        want = flags.get("expect_ops", {})
        for kind, positive in want.items():
            assert (fused.op_counts[kind] > 0) == positive, (kind, fused.op_counts)
        plx.shutdown()  # unmaps and unlinks the shared-memory workspaces


GRIDS = [(2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 2, 1), (1, 2, 2), (2, 1, 2), (4, 1, 1), (1, 1, 4)]


@pytest.mark.parametrize("grid", GRIDS)
def test_grids_three_layers(grid):
    world = grid[0] * grid[1] * grid[2]
    run_distributed(_worker, world, grid, 3, True, 61, 10, 5, 12, True, {})


@pytest.mark.parametrize("grid", [(2, 2, 2), (4, 2, 1)])
def test_eight_ranks(grid):
    run_distributed(_worker, 8, grid, 3, True, 53, 9, 7, 8, True, {})


@pytest.mark.parametrize("num_layers", [1, 2, 4])
def test_layer_counts_cover_rotation(num_layers):
    run_distributed(_worker, 4, (2, 1, 2), num_layers, True, 50, 6, 4, 8, True, {})


@pytest.mark.parametrize("grid", [(2, 2, 1), (1, 2, 2), (2, 1, 2), (4, 1, 1)])
@pytest.mark.parametrize("order", ["combine_first", "aggregate_first"])
def test_layer_order(grid, order):
    world = grid[0] * grid[1] * grid[2]
    run_distributed(_worker, world, grid, 3, True, 57, 10, 5, 16, True, {"order": order})


def test_combine_first_eight_ranks_four_layers():
    run_distributed(_worker, 8, (2, 2, 2), 4, True, 53, 9, 7, 16, True, {"order": "combine_first"})


def test_single_permutation_and_unfused_layers():
    run_distributed(_worker, 4, (1, 2, 2), 3, False, 47, 7, 3, 8, False, {})


def test_channel_alignment_padding():
    run_distributed(_worker, 2, (1, 2, 1), 2, True, 40, 10, 5, 12, True, {"align": 8})


def test_blocked_and_overlapped_aggregation():
    run_distributed(_worker, 2, (2, 1, 1), 2, True, 64, 8, 4, 8, True, {"block": True})
    run_distributed(_worker, 2, (2, 1, 1), 2, True, 64, 8, 4, 8, True, {"block": True, "overlap": True})


def test_tuned_gemms():
    run_distributed(_worker, 2, (1, 1, 2), 2, True, 40, 8, 4, 8, True, {"tune": True})


def test_single_process_matches_oracle():
    import plexus_b200 as plx
    from plexus_b200.models.cross_entropy import parallel_cross_entropy
    from plexus_b200.models.net import Net
    from plexus_b200.utils.dataloader import DataLoader

    plx.init(1, 1, 1, device="cpu", dtype=torch.float64, channel_align=1)
    data, nc = small_processed_graph(n=70, e=300, f=9, c=4, seed=2)
    adj, feats, labels, N, F, C = DataLoader(None, 3, data=(data, nc), dtype=torch.float64).load()
    model = Net(3, F, 16, C, seed=4).double()
    loss = parallel_cross_entropy(model(feats, adj), labels, 3, N, C)
    loss.backward()
    ref_loss, ref_gw, ref_gx, _ = oracle(data, nc, 3, 16, seed=4)
    assert torch.allclose(loss.detach(), ref_loss, rtol=1e-10)
    assert torch.allclose(feats.grad.view(N, F), ref_gx, rtol=1e-8, atol=1e-12)
    for l, layer in enumerate(model.layers):
        assert torch.allclose(layer.weight.grad.view_as(ref_gw[l]), ref_gw[l], rtol=1e-8, atol=1e-12)


def _axis_host_check(rank, world, split):
    import os

    import torch.distributed as dist
    from plexus_b200.parallel import symm

    os.environ["PLEXUS_HOST_ID"] = f"node{rank // 2}" if split else "node0"
    ax = symm.AxisComm(dist.group.WORLD)
    assert ax.p == world and ax.rank == rank and ax.peers == [q for q in range(world) if q != rank]
    assert ax.same_host == (not split)
    if split:
        # no peer-memory workspace may be requested for an axis that spans hosts
        try:
            ax.ensure(1024)
        except RuntimeError as e:
            assert "spans hosts" in str(e)
        else:
            raise AssertionError("ensure() must refuse")


@pytest.mark.parametrize("split", [False, True])
def test_peer_memory_axes_are_limited_to_one_host(split):
    run_distributed(_axis_host_check, 4, split)


EMU = {"emulate_peer_memory": True}


@pytest.mark.parametrize("grid", [(2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 1, 2), (2, 2, 1), (1, 2, 2), (4, 1, 1),
                                  (2, 2, 2), (1, 4, 2), (8, 1, 1)])
def test_fused_host_code_on_emulated_peer_memory_one_shot(grid):
    """symm.py / fused.py (slots, flags, op parity, workspace growth) with the one-shot push on every axis."""
    world = grid[0] * grid[1] * grid[2]
    # 64 nodes divide by every axis size, so a depth axis reduce-scatters the feature gradient
    expect = {"one_shot": True, "two_shot": False, "library": False, "reduce_scatter": grid[2] > 1}
    run_distributed(_worker, world, grid, 3, True, 64, 10, 5, 12, False,
                    dict(EMU, one_shot_ranks=8, expect_ops=expect))


@pytest.mark.parametrize("grid", [(2, 1, 1), (1, 1, 4), (1, 4, 1), (2, 2, 2), (4, 2, 1), (1, 1, 8), (2, 4, 1)])
def test_fused_host_code_on_emulated_peer_memory_two_shot(grid):
    """Every message through the two-shot form: reduce-scatter push, segment reduce + broadcast, landing."""
    world = grid[0] * grid[1] * grid[2]
    expect = {"one_shot": False, "two_shot": True, "library": False}
    run_distributed(_worker, world, grid, 3, True, 53, 9, 7, 8, False,
                    dict(EMU, two_shot=True, small_bytes=0, one_shot_ranks=1, expect_ops=expect))


@pytest.mark.parametrize("mode", ["pipeline", "in_kernel"])
@pytest.mark.parametrize("grid", [(2, 1, 1), (1, 1, 2), (2, 2, 2), (1, 4, 1)])
def test_fused_host_code_flag_free_forms(grid, mode):
    """The one-shot forms whose receive side needs no flags (sentinel-kept slots): reduce kernel on row
    chunks (pipeline) and reduction inside the compute kernel (in_kernel), on the emulated peer memory."""
    world = grid[0] * grid[1] * grid[2]
    key = "pipelined" if mode == "pipeline" else "in_kernel"
    run_distributed(_worker, world, grid, 3, True, 300, 10, 5, 12, False,
                    dict(EMU, one_shot_ranks=8, small_bytes=0, pipeline_min_bytes=4096, **{mode: True},
                         expect_ops={"one_shot": True, key: True, "library": False}))


@pytest.mark.parametrize("grid,max_bytes", [((1, 1, 4), None), ((1, 4, 1), None), ((4, 2, 1), None), ((1, 1, 8), None),
                                            ((2, 2, 2), None), ((4, 1, 1), 8000), ((1, 3, 1), None)])
def test_fused_host_code_segment_reduce_on_a_symmetric_buffer(grid, max_bytes):
    """Every matrix all-reduce through the symmetric buffer: partials written locally, each rank reduces
    its row segment and broadcasts it (what the switch does for the multimem kernel), flagged copy out;
    in row chunks, and in row blocks when the message limit is small."""
    world = grid[0] * grid[1] * grid[2]
    flags = dict(EMU, segment_reduce=True, small_bytes=0, one_shot_ranks=1, pipeline_min_bytes=4096,
                 expect_ops={"segment_reduce": True, "library": False, "two_shot": False})
    if max_bytes:
        flags.update(max_message_bytes=max_bytes, row_block_multiple=8)
    run_distributed(_worker, world, grid, 3, True, 300, 10, 5, 12, False, flags)


@pytest.mark.parametrize("grid,layers", [((2, 1, 1), 1), ((1, 2, 1), 3), ((1, 1, 2), 2), ((2, 2, 2), 3), ((1, 4, 1), 3),
                                         ((1, 4, 2), 2), ((8, 1, 1), 1)])
def test_cross_entropy_exchange_inside_the_kernels(grid, layers):
    """Class-sharded loss with the row statistics pushed by the statistics kernel and read (after its
    flag barrier) by the combine kernel, on the emulated peer memory.  The class axis (x / z / y for
    1 / 2 / 3 layers) has 2, 4 or 8 ranks; with 5 classes some shards hold padding only."""
    world = grid[0] * grid[1] * grid[2]
    run_distributed(_worker, world, grid, layers, True, 64, 10, 5, 12, False,
                    dict(EMU, one_shot_ranks=8, xent_exchange=True, expect_ops={"xent_exchange": True}))


def test_segment_reduce_with_fewer_rows_than_ranks():
    """9 nodes on an 8-rank axis: most ranks own an empty segment and only take part in the barriers."""
    flags = dict(EMU, segment_reduce=True, small_bytes=0, one_shot_ranks=1,
                 expect_ops={"segment_reduce": True, "library": False})
    run_distributed(_worker, 8, (1, 1, 8), 2, True, 9, 3, 2, 4, False, flags)
    run_distributed(_worker, 8, (8, 1, 1), 2, True, 9, 3, 2, 4, False, flags)


def test_fused_host_code_default_policy_mixes_push_and_library_paths():
    """Default thresholds on a 4-rank axis: small messages pushed, large ones reduced by the library."""
    run_distributed(_worker, 4, (4, 1, 1), 2, True, 61, 10, 5, 12, False,
                    dict(EMU, small_bytes=3000, expect_ops={"one_shot": True, "library": True, "two_shot": False}))


@pytest.mark.parametrize("num_layers,double_perm", [(1, True), (2, False), (4, True), (5, False)])
def test_fused_host_code_layer_counts_and_permutations(num_layers, double_perm):
    """Role rotation wrap-around and both permutation schemes through the emulated two-shot path."""
    run_distributed(_worker, 4, (2, 1, 2), num_layers, double_perm, 50, 6, 4, 8, False,
                    dict(EMU, two_shot=True, small_bytes=0, one_shot_ranks=1))


def _random_configs(seed, count):
    import random

    rng = random.Random(seed)
    grids = [(2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 2, 1), (1, 2, 2), (2, 1, 2), (4, 1, 1), (1, 4, 1), (1, 1, 4),
             (2, 2, 2), (4, 2, 1), (1, 4, 2), (2, 1, 4), (8, 1, 1), (1, 8, 1), (1, 1, 8)]
    out = []
    for _ in range(count):
        flags = {}
        if rng.random() < 0.3:
            flags["align"] = rng.choice([2, 8])
        if rng.random() < 0.3:
            flags["order"] = rng.choice(["aggregate_first", "auto"])
        mode = rng.random()
        if mode < 0.35:
            flags.update(EMU, one_shot_ranks=8)
        elif mode < 0.7:
            flags.update(EMU, two_shot=True, small_bytes=0, one_shot_ranks=1)
        out.append((rng.choice(grids), rng.choice([1, 2, 3, 4, 5]), rng.choice([True, False]),
                    rng.choice([9, 17, 33, 50, 64, 97]), rng.choice([1, 3, 7, 10, 16]), rng.choice([2, 3, 5, 9]),
                    rng.choice([1, 4, 6, 12]), rng.choice([True, False]), flags))
    return out


@pytest.mark.parametrize("cfg", _random_configs(2024, 10), ids=lambda c: "x".join(map(str, c[0])) + f"-L{c[1]}-n{c[3]}")
def test_random_configurations(cfg):
    """Seeded random draws of grid, depth, sizes (down to 9 nodes on 8 ranks, 1 feature, 1 hidden
    channel), permutation scheme, layer fusion, alignment, order and collective path."""
    grid, layers, double_perm, n, f, c, hidden, fuse, flags = cfg
    run_distributed(_worker, grid[0] * grid[1] * grid[2], grid, layers, double_perm, n, f, c, hidden, fuse, flags)


def _skip_worker(rank, world, emulate):
    import plexus_b200 as plx
    from plexus_b200.models.cross_entropy import parallel_cross_entropy
    from plexus_b200.models.net import Net
    from plexus_b200.parallel import collectives as coll
    from plexus_b200.utils.dataloader import DataLoader

    comm = None
    if emulate:
        from plexus_b200.parallel import emulator

        emulator.enable()
        comm = "fused"
    plx.init(2, 2, 2, device="cpu", dtype=torch.float64, comm=comm)
    data, nc = small_processed_graph(n=64, e=300, f=10, c=5, seed=5)
    adj, feats, labels, N, F, C = DataLoader(None, 3, data=(data, nc), dtype=torch.float64).load()
    model = Net(3, F, 12, C, seed=11).double()
    coll.bytes_moved(reset=True)
    plx.runtime.flags.skip_collectives = True
    loss = parallel_cross_entropy(model(feats, adj), labels, 3, N, C)
    loss.backward()
    assert torch.isfinite(loss) and all(torch.isfinite(l.weight.grad).all() for l in model.layers)
    assert feats.grad.shape == feats.shape
    assert sum(coll.bytes_moved().values()) == 0      # nothing was handed to a collective
    plx.runtime.flags.skip_collectives = False
    plx.shutdown()


@pytest.mark.parametrize("emulate", [False, True])
def test_compute_only_mode_runs_the_same_shapes_without_communication(emulate):
    """``flags.skip_collectives`` (used to measure exposed communication) keeps every shape."""
    run_distributed(_skip_worker, 8, emulate)


def _dropout_worker(rank, world, grid):
    import plexus_b200 as plx
    from helpers import dense_adj
    from plexus_b200.models.cross_entropy import parallel_cross_entropy
    from plexus_b200.models.net import Net, SerialGCN, serial_loss
    from plexus_b200.utils.checkpoint import _cut_features, _cut_weight
    from plexus_b200.utils.dataloader import DataLoader

    plx.init(*grid, device="cpu", dtype=torch.float64)
    data, nc = small_processed_graph(n=61, e=300, f=10, c=5, seed=5)
    adj, feats, labels, N, F, C = DataLoader(None, 3, data=(data, nc), dtype=torch.float64).load()
    model = Net(3, F, 12, C, seed=11, dropout=0.4).double()
    assert not model.fuse_layers
    serial = SerialGCN(3, F, 12, C, seed=11, dtype=torch.float64)
    adjs = [dense_adj(data.edge_index, data.edge_weight, N).to_sparse(),
            dense_adj(data.edge_index_2, data.edge_weight_2, N).to_sparse()]
    for step in range(2):  # the masks change from step to step, identically on both sides
        feats.grad = None
        for p_ in model.parameters():
            p_.grad = None
        loss = parallel_cross_entropy(model(feats, adj), labels, 3, N, C)
        loss.backward()
        x = data.x.double().clone().requires_grad_()
        for w in serial.weights:
            w.grad = None
        ref = serial_loss(serial(x, adjs, dropout=0.4, seed=11, step=step), data.y, N)
        ref.backward()
        assert torch.allclose(loss.detach(), ref.detach(), rtol=1e-9), (step, loss.item(), ref.item())
        for l, layer in enumerate(model.layers):
            assert torch.allclose(layer.weight.grad, _cut_weight(layer, serial.weights[l].grad), rtol=1e-8, atol=1e-11)
        assert torch.allclose(feats.grad, _cut_features(x.grad, feats), rtol=1e-8, atol=1e-11)
    first = loss.item()
    model.eval()  # no dropout in evaluation mode
    with torch.no_grad():
        ev = parallel_cross_entropy(model(feats, adj), labels, 3, N, C).item()
        want = serial_loss(serial(data.x.double(), adjs), data.y, N).item()
    assert abs(ev - want) < 1e-9 and abs(ev - first) > 1e-6


@pytest.mark.parametrize("grid", [(1, 1, 1), (2, 1, 2), (2, 2, 2), (1, 4, 1)])
def test_dropout_masks_do_not_depend_on_the_grid(grid):
    """Net(dropout=p): every grid drops the same elements as the serial model with the same seed."""
    run_distributed(_dropout_worker, grid[0] * grid[1] * grid[2], grid)


@pytest.mark.parametrize("grid", [(2, 1, 1), (1, 2, 1), (1, 1, 2), (2, 2, 2)])
def test_fused_host_code_row_blocked_messages(grid):
    """A cap on the bytes per op splits every fused all-reduce in row blocks (one op each)."""
    world = grid[0] * grid[1] * grid[2]
    run_distributed(_worker, world, grid, 3, True, 61, 10, 5, 12, False,
                    dict(EMU, one_shot_ranks=8, max_message_bytes=1200, row_block_multiple=8,
                         expect_ops={"one_shot": True, "library": False, "row_blocked": True}))


def _gather_pieces_worker(rank, world):
    import plexus_b200 as plx
    from plexus_b200.parallel import emulator, fused

    emulator.enable()
    fused.MAX_MESSAGE_BYTES = 64  # 4 pieces of 64 bytes + a remainder
    grid = plx.init(world, 1, 1, device="cpu", comm="fused")
    g = grid.group("x")
    for n in (70, 16, 3):
        mine = torch.arange(n, dtype=torch.float32) + 1000 * rank
        got = fused.all_gather(mine, g)
        want = torch.cat([torch.arange(n, dtype=torch.float32) + 1000 * r for r in range(world)])
        assert torch.equal(got, want), n
    two_d = fused.all_gather(torch.full((5, 6), float(rank)), g)
    assert two_d.shape == (5 * world, 6) and torch.equal(two_d[5 * rank], torch.full((6,), float(rank)))
    emulator.ops.check_status()
    plx.shutdown()


def test_fused_all_gather_in_pieces():
    run_distributed(_gather_pieces_worker, 3)


def _replica_worker(rank, world):
    """One-shot sums on a 4-rank axis: every rank must add the partials in the same (group-rank)
    order, so the replicas of an all-reduced fp32 tensor are bitwise equal."""
    import torch.distributed as dist

    import plexus_b200 as plx
    from plexus_b200.parallel import emulator, fused

    emulator.enable()
    fused.ONE_SHOT_MAX_RANKS = 8
    grid = plx.init(world, 1, 1, device="cpu", comm="fused")
    g = grid.group("x")
    gen = torch.Generator().manual_seed(100 + rank)
    # magnitudes spread over many binades: a different summation order changes the last bits
    t = torch.randn(4096, generator=gen) * torch.exp(8 * torch.randn(4096, generator=gen))
    mine = t.clone()
    fused.all_reduce_f32(mine, g)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    assert all(torch.equal(everyone[0], e) for e in everyone)
    # and it is the sum in group-rank order
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t)
    want = torch.zeros_like(t)
    for p in parts:
        want = want + p
    assert torch.equal(mine, want)
    m = torch.randn(64, 16, generator=gen).to(torch.bfloat16)
    fused.all_reduce_bf16(m, g)
    every_m = [torch.empty_like(m) for _ in range(world)]
    dist.all_gather(every_m, m)
    assert all(torch.equal(every_m[0], e) for e in every_m)
    emulator.ops.check_status()
    plx.shutdown()


def test_one_shot_replicas_are_bitwise_equal_on_a_four_rank_axis():
    run_distributed(_replica_worker, 4)
