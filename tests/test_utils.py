"""Timers, timer report, log parser, matmul tuner, facade package, optimizer (CPU)."""

import math
import os

import pytest
import torch


def test_nested_timers_and_tree_report():
    from plexus_b200.utils.general import format_timer_tree, reduce_timer_data
    from plexus_b200.utils.timers import Timers

    t = Timers(enabled=True, use_cuda=False)
    t.start("epoch 0")
    t.start("gcn conv fwd")
    t.start("AGG = A * H")
    t.stop("AGG = A * H")
    t.stop("gcn conv fwd")
    t.start("gcn conv fwd")
    t.stop("gcn conv fwd")
    t.stop("epoch 0")
    times, counts = t.get_times()
    assert set(times) == {("epoch 0",), ("epoch 0", "gcn conv fwd"), ("epoch 0", "gcn conv fwd", "AGG = A * H")}
    assert counts[("epoch 0", "gcn conv fwd")] == 2
    assert t.get_times()[0] == {}  # reset
    with pytest.raises(RuntimeError):
        t.start("a")
        t.stop("b")
    text = format_timer_tree(reduce_timer_data(times))
    lines = [l for l in text.splitlines() if l.strip()]
    assert "epoch 0 | Max Time:" in lines[0] and lines[1].startswith("\t|--") and lines[2].startswith("\t\t|--")
    assert "Load Imbalance: 1.000" in lines[0]
    off = Timers(enabled=False)
    off.start("x")
    off.stop("y")  # disabled timers ignore everything
    assert off() is off  # usable as ``get_timers()`` and as ``get_timers``


def test_process_log_file_on_canned_log(tmp_path):
    from plexus_b200.utils.parse_results import extract_avg_time, process_log_file

    def block(scale):
        return "\n".join([
            f"|-- 'epoch {scale} | Max Time: 9.0 ms | Avg Time: 9.0 ms | Load Imbalance: 1.0'",
            f"\t|-- 'gcn conv fwd | Max Time: 5 ms | Avg Time: 5 ms | Load Imbalance: 1.0'",
            f"\t\t|-- 'AGG = A * H | Max Time: 1 ms | Avg Time: {1.0 * scale} ms | Load Imbalance: 1.0'",
            f"\t\t|-- 'all-reduce | Max Time: 1 ms | Avg Time: {0.5 * scale} ms | Load Imbalance: 1.0'",
            f"\t\t|-- 'OUT = AGG * W | Max Time: 1 ms | Avg Time: {0.25 * scale} ms | Load Imbalance: 1.0'",
            f"\t\t|-- 'gather | Max Time: 1 ms | Avg Time: {0.125 * scale} ms | Load Imbalance: 1.0'",
            f"\t|-- 'cross entropy fwd | Max Time: 1 ms | Avg Time: {2.0 * scale} ms | Load Imbalance: 1.0'",
            f"\t|-- 'reduce-scatter | Max Time: 1 ms | Avg Time: {0.0625 * scale} ms | Load Imbalance: 1.0'",
            "Epoch: 000, Train Loss: 1.0000",
        ])

    path = tmp_path / "log.txt"
    path.write_text(block(1) + "\n" + block(2) + "\n" + block(4) + "\n")
    assert extract_avg_time("x | Avg Time: 3.25 ms") == 3.25 and extract_avg_time("nothing") == 0
    epoch, comm = process_log_file(str(path), 1)
    per = (1.0 + 0.25) + (0.5 + 0.125 + 0.0625) + 2.0
    assert math.isclose(epoch, per * 3) and math.isclose(comm, (0.5 + 0.125 + 0.0625) * 3)
    epoch0, _ = process_log_file(str(path), 0)
    assert math.isclose(epoch0, per * (1 + 2 + 4) / 3)


def test_tuned_matmul_caches_choice_and_matches_plain():
    from plexus_b200 import runtime
    from plexus_b200.utils import matmul_tuning as mt

    a, b = torch.randn(30, 20), torch.randn(20, 10)
    runtime.flags.tune_gemm = False
    assert torch.allclose(mt.tuned_matmul(a, b, "site"), a @ b, atol=1e-5)
    runtime.flags.tune_gemm = True
    mt.matmul_to_index.clear()
    out = mt.tuned_matmul(a, b, "site")
    assert torch.allclose(out, a @ b, atol=1e-5) and "site" in mt.matmul_to_index
    assert 0 <= mt.matmul_to_index["site"] < len(mt.transpose_orders) == len(mt.change_layouts) == 8
    out = mt.tuned_matmul(a, torch.randn(30, 10), "site2", trans_a=True)
    assert out.shape == (20, 10)
    for i in range(8):
        assert torch.allclose(mt.matmul(a, b, mt.change_layouts[i], mt.transpose_orders[i]), a @ b, atol=1e-5)
    assert mt.time_gpu(lambda: a @ b, warmup=1, trials=2) > 0


def test_facade_package_exposes_reference_names():
    from plexus import plexus as plx
    from plexus.cross_entropy import parallel_cross_entropy
    from plexus.gcn_conv import GCNConv, GCNConvFunction, chunked_spmm_all_reduce, extract_csr_submatrix
    from plexus.utils.dataloader import DataLoader
    from plexus.utils.dataset import partition_graph_2d, preprocess_graph
    from plexus.utils.general import get_process_groups_info, pad_dimension, set_seed
    from plexus.utils.matmul_tuning import tuned_matmul

    with pytest.raises(AssertionError):
        plx.init(overlap_aggregation=True, block_aggregation=False)
    plx.init(1, 1, 1, block_aggregation=True, overlap_aggregation=True, tune_gemms=True, device="cpu")
    assert plx.block_agg and plx.overlap_agg and plx.tune_gemm
    assert get_process_groups_info(("x", "y", "z"))[0] == [1, 1, 1]
    assert pad_dimension(5, 4) == 8
    set_seed(3)
    layer = GCNConv(6, 4, 0)
    assert layer.weight.dim() == 1 and layer.weight.numel() == 24 and layer.gather_features
    assert dict(layer.named_parameters()).keys() == {"weight"}
    A = torch.eye(5).to_sparse_csr()
    assert extract_csr_submatrix(A, 1, 3).shape == (2, 5)


def test_csr_helpers():
    from plexus_b200.utils.general import analyze_csr_tensor

    A = torch.tensor([[0.0, 3.0], [4.0, 0.0]]).to_sparse_csr()
    nnz, fro = analyze_csr_tensor(A)
    assert nnz == 2 and math.isclose(fro, 5.0)


def test_fused_adamw_cpu_matches_torch_adamw():
    from plexus_b200.optim import FusedAdam, FusedAdamW

    torch.manual_seed(0)
    p1 = [torch.randn(50, requires_grad=True), torch.randn(7, 3, requires_grad=True)]
    p2 = [p.detach().clone().requires_grad_() for p in p1]
    o1 = FusedAdamW(p1, lr=1e-2, weight_decay=0.1)
    o2 = torch.optim.AdamW(p2, lr=1e-2, weight_decay=0.1)
    for _ in range(5):
        for a, b in zip(p1, p2):
            g = torch.randn_like(a)
            a.grad, b.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    for a, b in zip(p1, p2):
        assert torch.allclose(a, b, atol=1e-6)
    # bf16 parameter keeps an fp32 master copy
    q = torch.randn(64).to(torch.bfloat16).requires_grad_()
    o3 = FusedAdam([q], lr=1e-2, weight_decay=0.01)
    q.grad = torch.ones_like(q)
    o3.step()
    st = o3.state[q]
    assert st["master"].dtype == torch.float32 and torch.equal(q.detach(), st["master"].to(torch.bfloat16))
    sd = o3.state_dict()
    o3.load_state_dict(sd)


def test_metrics_sink(tmp_path):
    import json

    from plexus_b200.utils.metrics import MetricsSink, max_over_ranks

    path = tmp_path / "m" / "metrics.jsonl"
    s = MetricsSink(str(path))
    s.log(event="epoch", epoch=0, loss=1.5)
    s.close()
    rec = json.loads(path.read_text().strip())
    assert rec["loss"] == 1.5 and "ts" in rec
    assert max_over_ranks(2.5) == 2.5


def test_fused_layer_sweep_plans_cases_and_formats_the_table(capsys):
    """The sweep driver of the fused-layer benchmark: case list, memory filter, commands, table."""
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarking",
                        "fused_layer_sweep.py")
    spec = importlib.util.spec_from_file_location("fused_layer_sweep", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    # 16M rows x degree 512 does not fit one GPU; 1M x 8 x 64 is tiny
    assert mod.estimate_gb(16_000_000, 512, 1024, 1024, 8) > 180
    assert mod.estimate_gb(1_000_000, 8, 64, 64, 2) < 3
    records, skipped = mod.main(["--gpus", "4", "--rows", "1000000,16000000", "--degrees", "8,512", "--widths", "64",
                                 "--kinds", "rmat", "--dry_run"])
    out = capsys.readouterr().out
    assert records == [] and len(skipped) == 1
    assert skipped[0][0]["rows"] == 16_000_000 and skipped[0][0]["degree"] == 512
    cmds = [line for line in out.splitlines() if "fused_layer.py" in line]
    assert len(cmds) == 3 and all("--nproc-per-node=4" in c and "--master-addr 127.0.0.1" in c for c in cmds)
    assert "--rows 16000000 --degree 8 --width 64" in out
    table = mod.summarise([{"kind": "rmat", "rows": 1000000, "nnz_per_rank": 32_000_000, "width": 256,
                            "spmm_fused_ms": 2.471, "spmm_nccl_ms": 2.482, "spmm_fused_fraction_of_roofline": 0.98,
                            "gemm_fused_ms": 1.406, "gemm_nccl_ms": 1.624, "gemm_fused_fraction_of_roofline": 0.83}])
    assert "| rmat | 1000000 | 32 | 256 | 2.47 / 2.48 / - | 0.98 | 1.41 / 1.62 / - | 0.83 |" in table


def test_source_style():
    """Formatting check of the tracked sources (the reference's CI runs a formatter check; this is the
    same kind of gate without a third-party tool): Python lines up to 120 columns, native sources up
    to 132, no tabs, no trailing blanks, every file ends with one newline."""
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        files = subprocess.run(["git", "ls-files"], cwd=root, capture_output=True, text=True, check=True).stdout.split()
    except Exception:
        pytest.skip("not a git checkout")
    bad = []
    for rel in files:
        ext = os.path.splitext(rel)[1]
        if rel.startswith("baseline/_ref") or ext not in (".py", ".cu", ".cuh", ".h", ".cpp"):
            continue
        limit = 120 if ext == ".py" else 132
        with open(os.path.join(root, rel)) as f:
            text = f.read()
        if text and not text.endswith("\n"):
            bad.append(f"{rel}: no newline at the end")
        for n, line in enumerate(text.split("\n"), 1):
            asm_operands = ext != ".py" and ('"=r"(' in line or '"=f"(' in line or "%0, %1, %2" in line)
            if len(line) > limit and not asm_operands:  # operand lists of inline PTX are left alone
                bad.append(f"{rel}:{n}: {len(line)} columns")
            if "\t" in line:
                bad.append(f"{rel}:{n}: tab")
            if line != line.rstrip():
                bad.append(f"{rel}:{n}: trailing blank")
    assert not bad, "\n".join(bad[:40])
