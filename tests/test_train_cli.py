"""The training application end to end on CPU ranks (the 2-layer / 16,384-node plumbing config)."""

import json
import os
import re
import subprocess
import sys

import pytest

from helpers import ROOT


def _run(args, nproc, tmp_path, port):
    env = dict(os.environ, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "examples", "train.py"),
           "--backend", "gloo"] + args
    if nproc == 1:
        cmd = [sys.executable, os.path.join(ROOT, "examples", "train.py"), "--backend", "gloo"] + args
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def _losses(out):
    return [float(m) for m in re.findall(r"Epoch: \d+, Train Loss: ([0-9.]+)", out)]


def test_two_rank_grid_matches_serial_run_and_logs_parse(tmp_path):
    # 2-layer GCN, fp32, R-MAT 16,384 nodes / ~262K undirected edges, 128 features, hidden 128,
    # 16 classes, Adam lr 0.01, 10 epochs; grid 2x1x1 over gloo versus one process
    common = ["--synthetic", "16384,262144,128,16", "--num_gcn_layers", "2", "--hidden_size", "128",
              "--lr", "0.01", "--num_epochs", "10", "--dtype", "fp32", "--seed", "1"]
    serial = _run(common, 1, tmp_path, 29611)
    metrics = tmp_path / "m.jsonl"
    par = _run(common + ["--G_intra_r", "2", "--metrics_file", str(metrics), "--eval"], 2, tmp_path, 29612)
    ls, lp = _losses(serial), _losses(par)
    assert len(ls) == len(lp) == 10
    assert all(abs(a - b) <= 2e-4 for a, b in zip(ls, lp)), (ls, lp)
    assert lp[-1] < lp[0]
    # the timer tree of the run parses with the reference-compatible log parser
    sys.path.insert(0, ROOT)
    from plexus_b200.utils.parse_results import process_log_file

    log = tmp_path / "par.log"
    log.write_text(par)
    epoch_ms, comm_ms = process_log_file(str(log), 2)
    assert epoch_ms > 0 and 0 < comm_ms < epoch_ms
    recs = [json.loads(l) for l in metrics.read_text().splitlines()]
    assert recs[0]["event"] == "start" and recs[0]["grid"] == [2, 1, 1]
    assert recs[0]["nnz"] > 2 * 200000 and recs[0]["model_epoch_ms"]["total"] > 0
    assert recs[-1]["collective_bytes"]["all-reduce"] > 0
    assert recs[-1]["event"] == "epoch" and 0.0 <= recs[-1]["acc_train"] <= 1.0


def test_resume_from_checkpoint_and_auto_grid(tmp_path):
    base = ["--synthetic", "600,4000,12,4", "--num_gcn_layers", "3", "--hidden_size", "16", "--seed", "2",
            "--dtype", "fp32", "--checkpoint_dir", str(tmp_path / "ck")]
    full = _losses(_run(base + ["--num_epochs", "4"], 1, tmp_path, 29613))
    os.system(f"rm -rf {tmp_path / 'ck'}")
    first = _losses(_run(base + ["--num_epochs", "2", "--checkpoint_every", "2"], 1, tmp_path, 29614))
    rest = _losses(_run(base + ["--num_epochs", "4", "--resume"], 1, tmp_path, 29615))
    assert len(first) == 2 and len(rest) == 2
    assert all(abs(a - b) < 1e-4 for a, b in zip(full, first + rest)), (full, first, rest)
    out = _run(["--synthetic", "600,4000,12,4", "--grid", "auto", "--num_epochs", "1", "--dtype", "fp32"], 2,
               tmp_path, 29616)
    assert "cost models chose grid" in out


def test_rank_local_synthetic_shards_train_like_one_process(tmp_path):
    """--sharded_synthetic: no rank builds the global graph, yet 4 ranks follow the 1-rank losses."""
    base = ["--synthetic", "900,6000,12,5", "--sharded_synthetic", "--num_gcn_layers", "3", "--hidden_size", "16",
            "--seed", "3", "--dtype", "fp32", "--num_epochs", "3", "--lr", "0.01"]
    one = _losses(_run(base, 1, tmp_path, 29617))
    four = _losses(_run(base + ["--G_intra_r", "2", "--G_intra_d", "2"], 4, tmp_path, 29618))
    assert len(one) == len(four) == 3
    assert all(abs(a - b) <= 2e-4 for a, b in zip(one, four)), (one, four)


_CLEAN = {}


def _clean_two_rank_losses(tmp_path, base):
    """Losses of the uninterrupted 2-rank run (computed once for both supervisor tests)."""
    if "losses" not in _CLEAN:
        _CLEAN["losses"] = _losses(_run(base + ["--G_intra_r", "2"], 2, tmp_path, 29621))
    return _CLEAN["losses"]


def test_a_wait_that_gave_up_stops_the_run_before_the_next_checkpoint(tmp_path):
    """Emulated peer memory on two CPU ranks; the status words get a TIMEOUT record before epoch 2
    (what a kernel leaves when a bounded wait runs out).  The check after the step must end the run
    with an error, and the checkpoint due after epoch 2 must not exist: the published one stays
    that of epoch 1."""
    args = ["--synthetic", "600,4000,12,4", "--num_gcn_layers", "3", "--hidden_size", "16", "--seed", "2",
            "--dtype", "fp32", "--G_intra_d", "2", "--comm", "fused", "--num_epochs", "4",
            "--checkpoint_dir", str(tmp_path / "ck"), "--checkpoint_every", "1"]
    env = dict(os.environ, OMP_NUM_THREADS="2", PLEXUS_EMULATE_PEER_MEMORY="1", PLEXUS_INJECT_FAILURE="0:2:status")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29619", os.path.join(ROOT, "examples", "train.py"),
           "--backend", "gloo"] + args
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(tmp_path))
    assert r.returncode != 0
    assert "PlexusCommTimeout" in r.stderr + r.stdout
    assert len(_losses(r.stdout)) == 2  # epochs 0 and 1 were reported, epoch 2 was not
    meta = json.loads((tmp_path / "ck" / "meta.json").read_text())
    assert meta["epoch"] == 1
    # the healthy rank may have started its own file of epoch 2; the failed rank wrote none and the
    # save was never published
    assert not (tmp_path / "ck" / "step_00000002" / "rank0.pt").exists()


def test_supervisor_restarts_from_the_last_checkpoint_after_a_lost_rank(tmp_path):
    """Rank 1 exits before epoch 2 (host-side injection); the supervisor resumes and the losses of the
    interrupted run continue exactly where an uninterrupted run goes."""
    base = ["--synthetic", "600,4000,12,4", "--num_gcn_layers", "3", "--hidden_size", "16", "--seed", "2",
            "--dtype", "fp32", "--num_epochs", "4", "--backend", "gloo"]
    clean = _clean_two_rank_losses(tmp_path, base)
    env = dict(os.environ, OMP_NUM_THREADS="2", PLEXUS_INJECT_FAILURE="1:2:exit")
    cmd = [sys.executable, os.path.join(ROOT, "examples", "supervise.py"), "--nproc", "2", "--max_restarts", "2",
           "--master_port", "29630", "--"] + base + ["--G_intra_r", "2", "--checkpoint_dir", str(tmp_path / "ck"),
                                                      "--checkpoint_every", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "injected failure: exiting before epoch 2" in r.stdout
    assert "[supervise] attempt 0 ended with exit code" in r.stdout and "finished after 1 restart(s)" in r.stdout
    got = _losses(r.stdout)
    assert len(got) == 4, r.stdout[-2000:]          # epochs 0, 1 from the first attempt, 2, 3 after the restart
    assert all(abs(a - b) < 1e-4 for a, b in zip(clean, got)), (clean, got)


def test_supervisor_can_restart_on_a_different_grid(tmp_path):
    """After the failure the job continues on another grid shape from the grid-independent
    checkpoint that is written next to the sharded one."""
    base = ["--synthetic", "600,4000,12,4", "--num_gcn_layers", "3", "--hidden_size", "16", "--seed", "2",
            "--dtype", "fp32", "--num_epochs", "4", "--backend", "gloo"]
    clean = _clean_two_rank_losses(tmp_path, base)
    env = dict(os.environ, OMP_NUM_THREADS="2", PLEXUS_INJECT_FAILURE="0:2:raise")
    cmd = [sys.executable, os.path.join(ROOT, "examples", "supervise.py"), "--nproc", "2", "--max_restarts", "1",
           "--master_port", "29650", "--restart_grid", "1x1x2", "--"] + base + [
        "--grid", "2x1x1", "--checkpoint_dir", str(tmp_path / "ck"), "--consolidated", str(tmp_path / "full.pt"),
        "--checkpoint_every", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "resumed from the consolidated checkpoint at epoch 2 on grid (1, 1, 2)" in r.stdout
    got = _losses(r.stdout)
    assert len(got) == 4, r.stdout[-2000:]
    assert all(abs(a - b) < 2e-4 for a, b in zip(clean, got)), (clean, got)


def test_grid_sweep_tool_runs_every_grid_on_one_generated_graph(tmp_path):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
           "--master-addr", "127.0.0.1", "--master-port", "29661", os.path.join(ROOT, "benchmarking", "grid_sweep.py"),
           "--backend", "gloo", "--dtype", "fp32", "--nodes", "500", "--edges", "3000", "--features", "12",
           "--hidden", "16", "--classes", "4", "--grids", "4x1x1,2x2x1,1x2x2", "--steps", "2", "--warmup", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=str(tmp_path),
                       env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    recs = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [tuple(x["grid"]) for x in recs[:3]] == [(4, 1, 1), (2, 2, 1), (1, 2, 2)]
    # same graph, same seed, same initial weights: the loss after 3 epochs does not depend on the grid
    assert max(x["loss"] for x in recs[:3]) - min(x["loss"] for x in recs[:3]) < 1e-4
    assert sorted(map(tuple, recs[3]["ranking"])) == [(1, 2, 2), (2, 2, 1), (4, 1, 1)]
    assert all(x["epoch_ms"] > 0 and x["model_ms"] > 0 for x in recs[:3])
