"""Tall-skinny GEMM micro-benchmark: the three dense products of a GCN layer on one GPU.

    python benchmarking/gemm.py [--rows 1000000 --k 256 --n 256 --variants]

Times ``OUT = relu(AGG . W)`` (gemm_nt), ``gradAGG = gradOUT . W^T`` (gemm_nt) and
``gradW = AGG^T . gradOUT`` (gemm_tn) with CUDA events and reports the achieved fraction of the
measured HBM copy bandwidth and of the measured cuBLAS bf16 peak, next to ``torch.mm`` in fp32
(what the reference runs) and in bf16.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from plexus_b200.ops import cuda as opc  # noqa: E402
from plexus_b200.perf.comm_model import load_measured_peaks  # noqa: E402


def timed(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1_000_000)
    ap.add_argument("--k", type=int, default=256)
    ap.add_argument("--n", type=int, default=256)
    ap.add_argument("--variants", action="store_true", help="time every launch variant of gemm_nt")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    M, K, N = args.rows, args.k, args.n
    dev = torch.device("cuda")
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(K, N, device=dev) / K**0.5).to(torch.bfloat16)
    g = torch.randn(M, N, device=dev).to(torch.bfloat16)
    peaks = load_measured_peaks()
    hbm, tf = peaks.get("hbm_gbs", 6555.0), peaks.get("bf16_tflops", 1640.0)

    def report(name, ms, bytes_moved, flops):
        print(f"{name:34s} {ms:8.3f} ms  {bytes_moved / ms / 1e6:7.0f} GB/s = {bytes_moved / ms / 1e6 / hbm:4.2f} of "
              f"measured HBM copy, {flops / ms / 1e9:7.1f} TFLOP/s = {flops / ms / 1e9 / tf:4.2f} "
              f"of measured bf16 peak")

    io_fwd = (M * K + M * N) * 2
    fl = 2.0 * M * K * N
    report("gemm_nt  OUT = relu(AGG.W)", timed(lambda: opc.gemm(a, w, relu=True), iters=args.iters), io_fwd, fl)
    report("gemm_nt  gradAGG = gradOUT.W^T", timed(lambda: opc.gemm(g, w, trans_b=True), iters=args.iters), io_fwd, fl)
    report("gemm_tn  gradW = AGG^T.gradOUT",
           timed(lambda: opc.gemm(a, g, trans_a=True, out_dtype=torch.float32), iters=args.iters), io_fwd, fl)
    if args.variants:
        for i, v in enumerate(opc.GEMM_VARIANTS):
            report(f"gemm_nt variant {i} {v}", timed(lambda: opc.gemm(a, w, relu=True, variant=i), iters=args.iters),
                   io_fwd, fl)
    af, wf = a.float(), w.float()
    torch.backends.cuda.matmul.allow_tf32 = False
    report("torch.mm fp32 (reference path)", timed(lambda: torch.mm(af, wf), iters=args.iters), (M * K + M * N) * 4, fl)
    report("torch.mm bf16 (cuBLAS)", timed(lambda: torch.mm(a, w), iters=args.iters), io_fwd, fl)
    opc.check_status()


if __name__ == "__main__":
    main()
