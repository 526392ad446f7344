"""Sweep of the fused compute+collective micro-benchmark over rows x degree x width x graph kind.

    python benchmarking/fused_layer_sweep.py --gpus 8 \
        --rows 1000000,4000000,16000000 --degrees 8,32,128,512 --widths 64,256,1024 --kinds rmat,uniform \
        [--out sweep.jsonl] [--dry_run]

Runs ``benchmarking/fused_layer.py`` once per combination under ``torch.distributed.run`` (one process
per GPU, rendezvous on 127.0.0.1), collects the JSON line each run prints and ends with a table: per
case the fused SpMM + all-reduce and GEMM + all-reduce times (the default form for the group size;
the other forms are not timed here, their workspaces do not fit the large cases), the same with NCCL after the compute
kernel and (unless ``--skip_reference``) with the reference's fp32 cuSPARSE / cuBLAS + NCCL path, and
the fused time as a fraction of its roofline.  Combinations whose operands would not fit
``--max_gb`` per GPU (CSR block + dense operands + result + receive buffers) are skipped and listed.

The reference has no such sweep; its closest tool times one SpMM on one GPU (benchmarking/spmm.py).
"""

import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def estimate_gb(rows: int, degree: int, width: int, out_width: int, ranks: int) -> float:
    """Device memory one rank needs for a case (bf16 operands, int32 / fp32 CSR, fp32 copies of the
    reference path, peer-memory receive buffers), in GB."""
    nnz = rows * degree
    csr = nnz * 8 + rows * 4
    dense = (rows // max(1, ranks)) * width * 2 + rows * width * 2 + width * out_width * 2
    results = rows * width * 2 + rows * out_width * 2
    buffers = 2 * min(ranks, 2) * max(rows * width, rows * out_width) * 2 if ranks == 2 else \
        1.25 * max(rows * width, rows * out_width) * 2
    reference = nnz * 12 + (rows * width + rows * out_width) * 4 * 2
    return (csr + dense + 2 * results + buffers + reference) / 1e9


def cases(rows, degrees, widths, kinds):
    for kind in kinds:
        for r in rows:
            for d in degrees:
                for w in widths:
                    yield {"rows": r, "degree": d, "width": w, "kind": kind}


def command(case, gpus: int, port: int, iters: int, skip_reference: bool):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "fused_layer.py"),
           "--rows", str(case["rows"]), "--degree", str(case["degree"]), "--width", str(case["width"]),
           "--out_width", str(case["width"]), "--kind", case["kind"], "--iters", str(iters), "--forms", "none"]
    if skip_reference:
        cmd.append("--skip_reference")
    return cmd


def summarise(records):
    """Markdown table of the collected records (one per case)."""
    head = ("| kind | rows | degree | width | SpMM+AR fused / NCCL / reference ms | fraction of roofline | "
            "GEMM+AR fused / NCCL / reference ms | fraction of roofline |")
    lines = [head, "|---|---|---|---|---|---|---|---|"]

    def ms(rec, key):
        v = rec.get(key)
        return "-" if v is None else f"{v:.2f}"

    for r in records:
        lines.append(
            f"| {r.get('kind')} | {r.get('rows')} | {round(r.get('nnz_per_rank', 0) / max(1, r.get('rows', 1)))} | "
            f"{r.get('width')} | {ms(r, 'spmm_fused_ms')} / {ms(r, 'spmm_nccl_ms')} / {ms(r, 'spmm_reference_ms')} | "
            f"{r.get('spmm_fused_fraction_of_roofline', float('nan')):.2f} | "
            f"{ms(r, 'gemm_fused_ms')} / {ms(r, 'gemm_nccl_ms')} / {ms(r, 'gemm_reference_ms')} | "
            f"{r.get('gemm_fused_fraction_of_roofline', float('nan')):.2f} |")
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--rows", type=str, default="1000000,4000000,16000000")
    ap.add_argument("--degrees", type=str, default="8,32,128,512")
    ap.add_argument("--widths", type=str, default="64,256,1024")
    ap.add_argument("--kinds", type=str, default="rmat,uniform")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--max_gb", type=float, default=150.0, help="skip cases that need more per GPU")
    ap.add_argument("--timeout", type=float, default=600.0, help="seconds per case")
    ap.add_argument("--port", type=int, default=29600)
    ap.add_argument("--skip_reference", action="store_true")
    ap.add_argument("--out", type=str, default=None, help="append every record to this JSON-lines file")
    ap.add_argument("--dry_run", action="store_true", help="print the commands, run nothing")
    args = ap.parse_args(argv)

    def ints(text):
        return [int(v) for v in text.split(",") if v]

    records, skipped = [], []
    for i, case in enumerate(cases(ints(args.rows), ints(args.degrees), ints(args.widths),
                                   [k for k in args.kinds.split(",") if k])):
        need = estimate_gb(case["rows"], case["degree"], case["width"], case["width"], args.gpus)
        if need > args.max_gb:
            skipped.append((case, need))
            continue
        cmd = command(case, args.gpus, args.port + i % 50, args.iters, args.skip_reference)
        if args.dry_run:
            print(" ".join(cmd))
            continue
        try:
            out = subprocess.run(cmd, capture_output=True, text=True, timeout=args.timeout)
        except subprocess.TimeoutExpired:
            skipped.append((case, -1.0))
            continue
        rec = None
        for line in out.stdout.splitlines():
            if line.startswith("{"):
                try:
                    rec = json.loads(line)
                except ValueError:
                    pass
        if rec is None:
            skipped.append((case, -2.0))
            sys.stderr.write(out.stderr[-2000:])
            continue
        records.append(rec)
        print(json.dumps(rec), flush=True)
        if args.out:
            with open(args.out, "a") as f:
                f.write(json.dumps(rec) + "\n")
    if records:
        print(summarise(records))
    for case, need in skipped:
        why = {-1.0: "timed out", -2.0: "printed no record"}.get(need, f"needs about {need:.0f} GB per GPU")
        print(f"skipped {case}: {why}")
    return records, skipped


if __name__ == "__main__":
    main()
