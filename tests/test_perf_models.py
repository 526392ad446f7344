"""Cost models: golden values (hand-derived from the closed forms) and structure."""

import math

import pytest

from plexus_b200.perf import chooser, comm_model, comp_model, mem_model
from plexus_b200.perf.common import split_into_three_powers_of_two


def test_split_into_three_powers_of_two():
    assert split_into_three_powers_of_two(1) == [(1, 1, 1)]
    s = split_into_three_powers_of_two(8)
    assert len(s) == 10 and all(x * y * z == 8 for x, y, z in s)
    assert s[0] == (1, 1, 8) and s[-1] == (8, 1, 1)
    with pytest.raises(ValueError):
        split_into_three_powers_of_two(6)


def test_comm_model_single_layer_by_hand():
    # one layer, grid (2,1,1): outer = X = 2, inner = Y = 1, depth = Z = 1, bandwidth-agnostic (v1)
    N, D, Dn = 1000, 64, 32
    cost = comm_model.compute_config_costs(2, N, [D, Dn], "v1", "perlmutter")[(2, 1, 1)]
    elem = 4 / 1024**3
    agg = 2 * (2 - 1) / 2 * (N * D / 1) * elem  # all-reduce of AGG over outer, forward
    want = (agg + agg) * 1000  # the same all-reduce of gradAGG in backward; every other term has p = 1
    assert math.isclose(cost, want, rel_tol=1e-12)


def test_comm_model_golden_values():
    c = comm_model.compute_config_costs(8, 2449029, [100, 128, 128, 47], "v3", "perlmutter")
    first = list(c.items())[:3]
    assert first[0][0] == (4, 1, 2) and math.isclose(first[0][1], 69.08277956868172, rel_tol=1e-9)
    assert first[1][0] == (1, 4, 2) and math.isclose(first[1][1], 70.78599689627646, rel_tol=1e-9)
    assert list(c.values()) == sorted(c.values())
    f = comm_model.compute_config_costs(8, 2449029, [100, 128, 128, 47], "v3", "frontier")
    assert len(f) == 10 and all(v > 0 for v in f.values())


def test_get_bw_tables():
    g = comm_model.get_bw
    assert g(1, 2, 4, "v1", "perlmutter") == 1
    assert g(1, 4, 4, "v2", "perlmutter") == 200 and g(2, 4, 4, "v2", "perlmutter") == 50
    assert g(1, 4, 4, "v3", "perlmutter") == 225 and g(1, 8, 4, "v3", "perlmutter") == 66.59
    assert g(2, 4, 4, "v3", "perlmutter") == 66.59 / 2 and g(4, 2, 4, "v3", "perlmutter") == 66.59 / 4
    assert g(1, 8, 8, "v3", "frontier") == 135 and g(2, 4, 8, "v3", "frontier") == 72
    assert g(4, 2, 8, "v3", "frontier") == 36 and g(8, 2, 8, "v3", "frontier") == 5
    assert g(3, 2, 8, "v3", "b200_nvl8") == comm_model.B200_PORT_GBS  # placement does not matter


def test_b200_comm_model_prefers_balanced_grid_and_uses_bf16():
    c = comm_model.compute_config_costs(8, 2449029, [100, 256, 256, 47], "v3", "b200_nvl8")
    assert list(c.keys())[0] == (2, 2, 2)
    one = comm_model.compute_config_costs(1, 1000, [8, 8], "v3", "b200_nvl8")
    assert one[(1, 1, 1)] == 0.0


def test_comp_model_golden_and_symmetry():
    c = comp_model.comp_model(2449029, 123718280, 8, [100, 128, 128])
    k0, v0 = next(iter(c.items()))
    assert k0 == (2, 2, 2) and math.isclose(v0, 9312969914.570568, rel_tol=1e-9)
    assert math.isclose(c[(2, 1, 4)], c[(4, 1, 2)], rel_tol=1e-12)
    # single GPU, one layer: cost = sqrt(F) * (1 + 2 N / D)
    one = comp_model.comp_model(100, 1000, 1, [10])[(1, 1, 1)]
    assert math.isclose(one, (1000 * 10) ** 0.5 * (1 + 2 * 100 / 10), rel_tol=1e-12)


def test_mem_model_golden_and_by_hand():
    m = mem_model.compute_config_mem(8, 2449029, 123718280, [100, 128, 128, 47])
    k0, v0 = next(iter(m.items()))
    assert k0 == "X2Y2Z2" and math.isclose(v0, 5.828322818502784, rel_tol=1e-9)
    # one GPU, one layer, by hand (32-bit words)
    N, E, D0, D1 = 10, 40, 4, 2
    # the adjacency term counts min(3, len(D_list)) = 2 layer types, as the reference does
    words = 2 * 2 * (3 * E + 2 * N) + 4 * D0 * D1 + 2 * N * D0 + 2 * N * D1 + 4 * N * D0 + (N * D0 + D0 * D1) + 2 * N
    got = mem_model.compute_config_mem(1, N, E, [D0, D1])["X1Y1Z1"]
    assert math.isclose(got, words * 4 / 1024**3, rel_tol=1e-12)
    b = mem_model.compute_config_mem_b200(8, 2449029, 123718280, [100, 128, 128, 47])
    assert b["X2Y2Z2"] < m["X2Y2Z2"]
    # peer-memory workspaces: by hand for one 2-rank axis (Z: all-gather H0 / reduce-scatter gradH0 of
    # N*D0/(X*Y) elements, no all-reduce on Z with one layer) - 2 buffers x 2 slots of one rank's piece
    ws = mem_model.workspace_bytes(1, 1, 2, 1000, [16, 8])
    assert ws == 1024 + 2 * 2 * (1000 * 16 * 2 / 2)
    # a 4-rank axis: symmetric buffer (1.25 x message) + small slots; the row-block limit caps it
    big = mem_model.workspace_bytes(4, 1, 1, 10**7, [128, 128, 128])
    capped = mem_model.workspace_bytes(4, 1, 1, 10**7, [128, 128, 128], max_message_bytes=64 << 20)
    assert capped < big and capped <= 1024 + 1.25 * (64 << 20) + 8 * (64 << 20)
    without = mem_model.compute_config_mem_b200(8, 2449029, 123718280, [100, 128, 128, 47], workspaces=False)
    assert all(b[k] > without[k] for k in b)


def test_chooser_returns_valid_grids_and_respects_memory():
    grids = chooser.choose_grid(8, 2449029, 123718280, [100, 256, 256, 47])
    assert len(grids) == 10 and all(x * y * z == 8 for x, y, z in grids)
    assert chooser.choose_grid(1, 1000, 5000, [8, 8]) == [(1, 1, 1)]
    tiny = chooser.choose_grid(8, 10**9, 5 * 10**10, [128, 128, 128, 64], mem_limit_gb=1.0)
    assert tiny == [(2, 2, 2)]  # nothing fits: the grid that needs the least memory, alone


def test_chooser_counts_the_workspaces_under_the_message_limit(monkeypatch):
    """The 111M-node graph on 8 GPUs: with 2 GiB messages no grid fits 170 GB (the workspaces alone take
    20 GB), with 256 MB row blocks 2x2x2 does."""
    args = (8, 111059956, 3232000000, [128, 128, 128, 172])
    monkeypatch.delenv("PLEXUS_MAX_MESSAGE_BYTES", raising=False)
    assert chooser.choose_grid(*args) == [(2, 2, 2)]  # least memory, nothing fits
    monkeypatch.setenv("PLEXUS_MAX_MESSAGE_BYTES", str(256 << 20))
    grids = chooser.choose_grid(*args)
    assert grids[0] == (2, 2, 2) and len(grids) >= 2


def test_facade_modules_reexport_the_models():
    import performance.comm_model as pc
    import performance.comp_model as pp
    import performance.mem_model as pm

    assert pc.compute_config_costs is comm_model.compute_config_costs
    assert pp.comp_model is comp_model.comp_model and pm.compute_config_mem is mem_model.compute_config_mem


def test_epoch_model_tracks_the_measured_epochs():
    """Predicted epoch times of the headline config against the device-timed B200 measurements."""
    from plexus_b200.perf.epoch_model import predict_epoch_ms, rank_grids

    N, NNZ, D = 2449029, 123717823, [100, 256, 256, 47]
    measured = {(1, 1, 1): 29.88, (1, 1, 2): 22.77, (1, 2, 1): 21.21, (2, 1, 1): 21.47, (2, 2, 1): 14.65,
                (2, 1, 2): 15.53, (4, 2, 1): 12.02}
    pred = {}
    for grid, ms in measured.items():
        r = predict_epoch_ms(grid, N, NNZ, D, hbm_gbs=6555.0)
        pred[grid] = r["total"]
        assert abs(r["total"] - ms) < 0.05 * ms, (grid, r)
        assert abs(sum(v for k, v in r.items() if k != "total") - r["total"]) < 1e-9
    # the measured order of the grids of 2 and of 4 GPUs
    assert pred[(1, 2, 1)] < pred[(2, 1, 1)] < pred[(1, 1, 2)] and pred[(2, 2, 1)] < pred[(2, 1, 2)]
    one = predict_epoch_ms((1, 1, 1), N, NNZ, D, hbm_gbs=6555.0)
    assert one["exposed_comm"] == 0.0 and one["gather"] == 0.0 and one["spmm"] > 0.7 * one["total"]
    # the 3D grid beats the flat ones on 8 ranks
    ranked = rank_grids(8, N, NNZ, D)
    assert ranked[0][1] == (2, 2, 2)
    assert dict((g, t) for t, g in ranked)[(8, 1, 1)] > 1.3 * ranked[0][0]
    # the dense-degree graph on 8 GPUs (233K nodes, 115M nonzeros): measured 9.09 / 10.08 / 7.40 / 10.84 ms
    dense = {(2, 2, 2): 9.09, (8, 1, 1): 10.08, (1, 8, 1): 7.40, (1, 1, 8): 10.84}
    for grid, ms in dense.items():
        r = predict_epoch_ms(grid, 233000, 115032984, [602, 256, 256, 41], hbm_gbs=6555.0)
        assert abs(r["total"] - ms) < 0.25 * ms, (grid, r)


def test_chooser_models():
    N, NNZ, D = 2449029, 123717823, [100, 256, 256, 47]
    # default (epoch model): on 2 GPUs the measured order 1x2x1 < 2x1x1 < 1x1x2
    assert chooser.choose_grid(2, N, NNZ, D) == [(1, 2, 1), (2, 1, 1), (1, 1, 2)]
    assert chooser.choose_grid(8, N, NNZ, D)[0] == (2, 2, 2)
    ep = chooser.choose_grid(8, N, NNZ, D, model="epoch")
    assert ep[0] == (2, 2, 2) and len(ep) == 10  # every grid that fits
    # the volume ranking (the reference's way of combining its models)
    assert chooser.choose_grid(2, N, NNZ, D, model="volume")[0] == (1, 1, 2)
    assert chooser.choose_grid(4, N, NNZ, D, model="volume")[0] == (2, 1, 2)
    assert chooser.choose_grid(8, N, NNZ, D, model="volume")[0] == (2, 2, 2)


def test_link_measurements_come_from_a_file_and_can_be_replaced(tmp_path, monkeypatch):
    """The B200 link figures are data, not literals: the packaged file, or the one PLEXUS_LINK_MEASUREMENTS names."""
    import json

    m = comm_model.load_link_measurements()
    assert m["port_gbs"] == comm_model.B200_PORT_GBS and m["latency_us"][2] > 0
    assert {"port_gbs", "allreduce_bus_gbs", "switch_reduce_port_gbs", "hbm_gbs"} <= set(m)
    other = dict(m, port_gbs=900.0, latency_us={"1": 0, "2": 1, "4": 2, "8": 3})
    path = tmp_path / "links.json"
    path.write_text(json.dumps(other))
    monkeypatch.setenv("PLEXUS_LINK_MEASUREMENTS", str(path))
    assert comm_model.load_link_measurements()["port_gbs"] == 900.0
    # an all-reduce on a 2-rank axis: one message over the port + the 3-pass reduce through HBM + latency
    t = comm_model.b200_all_reduce_seconds(2, 512e6)
    want = 8e-6 + 512e6 / (comm_model.B200_PORT_GBS * 1e9) + 3 * 512e6 / (comm_model.B200_HBM_GBS * 1e9)
    assert math.isclose(t, want, rel_tol=1e-12)
    # larger axes: (1 + 1/p) x message at the switch-reduce rate + the copy out; cheaper per byte at p = 8 than at 4
    assert comm_model.b200_all_reduce_seconds(8, 512e6) < comm_model.b200_all_reduce_seconds(4, 512e6)
