"""Checkpoint/resume (sharded and grid-independent) and host-side failure detection (CPU, gloo)."""

import os
import subprocess
import sys
import time

import pytest
import torch
import torch.distributed as dist

from helpers import ROOT, run_distributed, small_processed_graph


def _setup(grid, layers=3, hidden=12, seed=21):
    import plexus_b200 as plx
    from plexus_b200.models.net import Net
    from plexus_b200.optim import FusedAdamW
    from plexus_b200.utils.dataloader import DataLoader

    plx.init(*grid, device="cpu", dtype=torch.float32, channel_align=1)
    data, nc = small_processed_graph(n=64, e=300, f=10, c=5, seed=8)
    adj, feats, labels, N, F, C = DataLoader(None, layers, data=(data, nc), dtype=torch.float32).load()
    model = Net(layers, F, hidden, C, seed=seed)
    opt = FusedAdamW(list(model.parameters()) + [feats], lr=1e-2)
    return plx, model, opt, adj, feats, labels, N, F, C


def _step(model, opt, adj, feats, labels, N, C, layers=3):
    from plexus_b200.models.cross_entropy import parallel_cross_entropy

    opt.zero_grad(set_to_none=True)
    loss = parallel_cross_entropy(model(feats, adj), labels, layers, N, C)
    loss.backward()
    opt.step()
    return loss.item()


def _sharded_worker(rank, world, grid, ckdir):
    from plexus_b200.utils import checkpoint as ck

    plx, model, opt, adj, feats, labels, N, F, C = _setup(grid)
    for _ in range(2):
        _step(model, opt, adj, feats, labels, N, C)
    ck.save_sharded(ckdir, model, opt, feats, epoch=1)
    want = [_step(model, opt, adj, feats, labels, N, C) for _ in range(2)]
    plx.shutdown()
    # fresh model + optimizer, resume
    plx, model, opt, adj, feats, labels, N, F, C = _setup(grid, seed=99)
    assert ck.load_sharded(ckdir, model, opt, feats) == 2
    got = [_step(model, opt, adj, feats, labels, N, C) for _ in range(2)]
    assert all(abs(a - b) < 1e-6 for a, b in zip(want, got)), (want, got)
    assert set(model.state_dict().keys()) == {f"layers.{l}.weight" for l in range(3)}


def test_sharded_checkpoint_resume(tmp_path):
    run_distributed(_sharded_worker, 2, (2, 1, 1), str(tmp_path / "ck"))
    assert (tmp_path / "ck" / "meta.json").exists()
    assert (tmp_path / "ck" / "step_00000001" / "rank1.pt").exists()
    assert not [f for _, _, fs in os.walk(tmp_path / "ck") for f in fs if ".tmp" in f]


def _save_consolidated_worker(rank, world, grid, path, out):
    from plexus_b200.utils import checkpoint as ck

    plx, model, opt, adj, feats, labels, N, F, C = _setup(grid)
    for _ in range(2):
        _step(model, opt, adj, feats, labels, N, C)
    ck.save_consolidated(path, model, opt, feats, N, F, epoch=1)
    from plexus_b200.models.cross_entropy import parallel_cross_entropy

    with torch.no_grad():
        at_save = parallel_cross_entropy(model(feats, adj), labels, 3, N, C).item()
    nxt = [_step(model, opt, adj, feats, labels, N, C) for _ in range(2)]
    if rank == 0:
        torch.save(nxt, out)
        torch.save(at_save, out + ".loss")


def _load_consolidated_worker(rank, world, grid, path, out):
    from plexus_b200.utils import checkpoint as ck

    plx, model, opt, adj, feats, labels, N, F, C = _setup(grid, seed=77)
    assert ck.load_consolidated(path, model, opt, feats) == 2
    got = [_step(model, opt, adj, feats, labels, N, C) for _ in range(2)]
    want = torch.load(out)
    assert all(abs(a - b) < 2e-5 for a, b in zip(want, got)), (want, got)


def test_consolidated_checkpoint_resumes_on_a_different_grid(tmp_path):
    path, out = str(tmp_path / "full.pt"), str(tmp_path / "next.pt")
    run_distributed(_save_consolidated_worker, 2, (2, 1, 1), path, out)
    run_distributed(_load_consolidated_worker, 4, (1, 2, 2), path, out)
    run_distributed(_load_consolidated_worker, 1, (1, 1, 1), path, out)
    # the same file gives a single-process model for evaluation: its loss on the processed graph
    # equals the parallel model's loss at the moment of saving
    from helpers import dense_adj
    from plexus_b200.models.net import SerialGCN, serial_loss

    model, feats = SerialGCN.from_consolidated(path, dtype=torch.float64)
    data, nc = small_processed_graph(n=64, e=300, f=10, c=5, seed=8)
    adjs = [dense_adj(data.edge_index, data.edge_weight, 64).to_sparse(),
            dense_adj(data.edge_index_2, data.edge_weight_2, 64).to_sparse()]
    with torch.no_grad():
        loss = serial_loss(model(feats, adjs), data.y, 64).item()
    assert abs(loss - torch.load(out + ".loss")) < 2e-5


def test_truncated_or_mismatched_checkpoint_is_rejected(tmp_path):
    from plexus_b200.utils import checkpoint as ck

    plx, model, opt, adj, feats, labels, N, F, C = _setup((1, 1, 1))
    _step(model, opt, adj, feats, labels, N, C)
    d = str(tmp_path / "ck")
    ck.save_sharded(d, model, opt, feats, epoch=0)
    f0 = os.path.join(d, "step_00000000", "rank0.pt")
    blob = open(f0, "rb").read()
    open(f0, "wb").write(blob[: len(blob) // 2])  # a damaged file under the published name
    with pytest.raises(ck.CheckpointError, match="cannot read"):
        ck.load_sharded(d, model, opt, feats)
    os.remove(os.path.join(d, "meta.json"))
    with pytest.raises(ck.CheckpointError, match="meta.json missing"):
        ck.load_sharded(d, model, opt, feats)
    ck.save_sharded(d, model, opt, feats, epoch=0)
    import json

    meta = json.load(open(os.path.join(d, "meta.json")))
    meta["grid"] = [2, 1, 1]
    json.dump(meta, open(os.path.join(d, "meta.json"), "w"))
    with pytest.raises(ck.CheckpointError, match="grid"):
        ck.load_sharded(d, model, opt, feats)


def test_interrupted_save_keeps_the_previous_checkpoint(tmp_path):
    """A save that dies before publishing (rank files of the new epoch exist, meta.json still names
    the old one) must not be picked up, and a rank file from another epoch placed under the
    published directory is rejected instead of being mixed in."""
    import shutil

    from plexus_b200.utils import checkpoint as ck

    plx, model, opt, adj, feats, labels, N, F, C = _setup((1, 1, 1))
    _step(model, opt, adj, feats, labels, N, C)
    d = str(tmp_path / "ck")
    ck.save_sharded(d, model, opt, feats, epoch=0)
    w0 = {k: v.clone() for k, v in model.state_dict().items()}
    meta_before = open(os.path.join(d, "meta.json")).read()
    _step(model, opt, adj, feats, labels, N, C)
    ck.save_sharded(d, model, opt, feats, epoch=1)
    # undo the publication of epoch 1: this is what the directory looks like when a rank died
    # after writing its epoch-1 file and before rank 0 replaced meta.json
    open(os.path.join(d, "meta.json"), "w").write(meta_before)
    assert ck.load_sharded(d, model, opt, feats) == 1
    assert all(torch.equal(v, w0[k]) for k, v in model.state_dict().items())
    # a later epoch's file under the published directory: refuse to mix epochs
    shutil.copy(os.path.join(d, "step_00000001", "rank0.pt"), os.path.join(d, "step_00000000", "rank0.pt"))
    with pytest.raises(ck.CheckpointError, match="inconsistent"):
        ck.load_sharded(d, model, opt, feats)


def test_sharded_save_prunes_old_steps(tmp_path):
    from plexus_b200.utils import checkpoint as ck

    plx, model, opt, adj, feats, labels, N, F, C = _setup((1, 1, 1))
    d = str(tmp_path / "ck")
    for e in range(4):
        ck.save_sharded(d, model, opt, feats, epoch=e)
    assert sorted(x for x in os.listdir(d) if x.startswith("step_")) == ["step_00000002", "step_00000003"]
    assert ck.load_sharded(d, model, opt, feats) == 4


# ------------------------------------------------------------------ failure detection
def _heartbeat_worker(rank, world, mode):
    from plexus_b200.parallel.watchdog import Heartbeat, PeerFailure

    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, prefix=f"hb-{mode}")
    hb.beat(0)
    hb.wait_for_peers(0, timeout_s=20)
    dist.barrier()  # everybody has seen step 0 before the failure is injected
    if mode == "exit":
        if rank == 1:
            hb.announce_exit("injected")  # a rank that leaves between steps
        else:
            t0 = time.time()
            with pytest.raises(PeerFailure) as e:
                while time.time() - t0 < 20:
                    hb.check_peers(max_age_s=30)
                    time.sleep(0.05)
            assert e.value.ranks == [1] and "exit" in str(e.value)
    elif mode == "stall":
        if rank == 1:
            time.sleep(1.5)  # never beats again within the limit
        else:
            hb.beat(1)
            with pytest.raises(PeerFailure) as e:
                hb.wait_for_peers(1, timeout_s=0.6)
            assert e.value.ranks == [1]
            # the peer's beat of step 0 is fresh enough for the age test but it lags behind step 1:
            # min_step catches it on its own, after the grace period only
            hb.check_peers(max_age_s=30, min_step=1, lag_grace_s=30)
            with pytest.raises(PeerFailure) as e:
                hb.check_peers(max_age_s=30, min_step=1, lag_grace_s=0.1)
            assert e.value.ranks == [1] and "below step 1" in str(e.value)
            time.sleep(0.5)
            with pytest.raises(PeerFailure):
                hb.check_peers(max_age_s=0.3)
    else:
        for step in range(1, 4):
            hb.beat(step)
            hb.wait_for_peers(step, timeout_s=20)
            hb.check_peers(max_age_s=30)


@pytest.mark.parametrize("mode", ["ok", "exit", "stall"])
def test_heartbeat_detects_lost_and_stalled_peers(mode):
    run_distributed(_heartbeat_worker, 2, mode)


def test_epoch_watchdog_fires_only_past_the_deadline():
    from plexus_b200.parallel.watchdog import EpochWatchdog

    fired = []
    with EpochWatchdog(0.2, on_timeout=fired.append, poll_s=0.02) as wd:
        wd.begin(0)
        time.sleep(0.05)
        wd.end()
        time.sleep(0.3)
        assert fired == []
        wd.begin(7)
        time.sleep(0.5)
        assert fired == [7] and wd.fired


def test_watchdog_default_action_exits_the_process():
    code = (
        "import sys, time; sys.path.insert(0, %r)\n"
        "from plexus_b200.parallel.watchdog import EpochWatchdog\n"
        "wd = EpochWatchdog(0.2); wd.begin(3); time.sleep(5); print('survived')\n" % ROOT
    )
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60)
    assert r.returncode == 43 and "survived" not in r.stdout and "step 3" in r.stdout


def test_rank_that_never_joins_ends_in_a_timeout_not_a_hang(tmp_path):
    """A collective with a missing peer must fail within the process-group timeout."""
    code = (
        "import sys, datetime, torch, torch.distributed as dist\n"
        "dist.init_process_group('gloo', init_method='file://%s', rank=0, world_size=2,\n"
        "                        timeout=datetime.timedelta(seconds=2))\n" % (tmp_path / "init")
    )
    t0 = time.time()
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode != 0 and time.time() - t0 < 100


def test_device_status_decoding():
    from plexus_b200.parallel.watchdog import PlexusCommTimeout, decode_status, raise_on_device_status

    ok = torch.zeros(8, dtype=torch.int32)
    raise_on_device_status(ok)
    st = torch.tensor([1, 1, 3, 42, 41, 0, 0, 0], dtype=torch.int32)
    assert "spmm_all_reduce" in decode_status(st.tolist()) and "expected 42, seen 41" in decode_status(st.tolist())
    with pytest.raises(PlexusCommTimeout):
        raise_on_device_status(st)
    assert int(st[0]) == 0  # cleared for the next step


def _silent_peer_worker(rank, world):
    """Rank 1 never runs its second collective: rank 0's bounded wait must end in a status word."""
    import plexus_b200 as plx
    from plexus_b200.parallel import emulator, fused, symm
    from plexus_b200.parallel.watchdog import PlexusCommTimeout

    emulator.enable()
    grid = plx.init(2, 1, 1, device="cpu", comm="fused")
    g = grid.group("x")
    t = torch.full((16,), float(rank + 1))
    fused.all_reduce_f32(t, g)                      # both ranks: sets up the workspace, op 1
    assert torch.equal(t, torch.full((16,), 3.0))
    ax = symm.axis_for(g)
    ax.timeout_ms = 300.0
    if rank == 0:
        u = torch.ones(16)
        t0 = time.time()
        fused.all_reduce_f32(u, g)                  # op 2: the peer never publishes its flag
        assert time.time() - t0 < 5.0
        with pytest.raises(PlexusCommTimeout, match="peer/slot 0, expected 2, seen 0"):
            emulator.ops.check_status()
        emulator.ops.check_status()                 # cleared; the rank is still usable
    dist.barrier()
    plx.shutdown()


def test_peer_that_never_raises_its_flag_ends_in_a_status_word():
    run_distributed(_silent_peer_worker, 2)
