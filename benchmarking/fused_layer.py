"""Fused compute+collective micro-benchmark along one grid axis (2 / 4 / 8 GPUs).

    torchrun --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 benchmarking/fused_layer.py \
        [--rows 1000000 --degree 32 --width 256 --kind rmat|uniform --out_width 256]

Every rank holds its own sparse block ``A_r`` (rows x rows/P, seeded) and dense operand and the
P ranks compute ``all_reduce_sum(A_r . H_r)`` and ``all_reduce_sum(X_r . W_r)``, the two patterns
of a 3D-parallel GCN layer (AGG over the outer axis, OUT over the inner axis).  Three paths:

* ``fused``     : this package's kernels, timed in the default form for the group size and in
                  every form explicitly: ``one_shot`` (the SpMM / tcgen05-GEMM epilogue stores each
                  row into every peer's receive slot over NVLink, a flagged kernel sums the slots),
                  ``two_shot`` (each row to its owner, which reduces and broadcasts its segment) and
                  ``segment`` (partials written into a symmetric buffer, each rank's segment summed
                  inside the NVSwitch by multimem loads and broadcast by multimem stores, in row
                  chunks on a side stream while the next chunk is computed; ``--segment_sweep``
                  also times other chunk counts and grid sizes of the reduce kernel);
* ``nccl``      : the same compute kernels followed by ``dist.all_reduce`` (NCCL);
* ``reference`` : what the reference executes: ``torch.sparse.mm`` / ``torch.mm`` in fp32
                  (cuSPARSE / cuBLAS) followed by an fp32 NCCL all-reduce.

Times are CUDA-event times, max over ranks.  The roofline time of a fused op is the slower of
FLOPs / measured bf16 GEMM peak and bytes that must cross NVLink / 770 GB/s per direction (measured
peer-copy bandwidth), with 2 (P-1)/P x message bytes for an all-reduce; for the SpMM the HBM
gather bound (nnz x row bytes / measured copy bandwidth) is reported as well.
"""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

NVLINK_GBS = 770.0


def timed(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1_000_000)
    ap.add_argument("--degree", type=int, default=32, help="mean nonzeros per row of the local block")
    ap.add_argument("--width", type=int, default=256, help="dense width D of the SpMM operand / GEMM K")
    ap.add_argument("--out_width", type=int, default=256, help="GEMM N")
    ap.add_argument("--kind", type=str, default="rmat", choices=["rmat", "uniform"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--skip_reference", action="store_true")
    ap.add_argument("--segment_sweep", action="store_true")
    ap.add_argument("--forms", type=str, default="one_shot,two_shot,segment",
                    help="fused forms to time explicitly besides the default one ('none': only the default; the "
                         "one-shot workspace is 2 x ranks x message bytes, too much for large cases on 8 ranks)")
    args = ap.parse_args()

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, p = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)

    import plexus_b200 as plx
    from plexus_b200 import ops
    from plexus_b200.data import graph_ops
    from plexus_b200.data.synthetic import rmat_edges, uniform_edges
    from plexus_b200.ops import cuda as opc
    from plexus_b200.parallel import fused
    from plexus_b200.perf.comm_model import load_measured_peaks

    grid = plx.init(p, 1, 1, comm="fused")
    group = grid.group("x")
    rows, cols = args.rows, max(1, args.rows // p)
    gen = rmat_edges if args.kind == "rmat" else uniform_edges
    r, c = gen(rows, rank * rows * args.degree, rows * args.degree, seed=7, device=dev)
    c = c % cols
    key = torch.unique(r * cols + c)
    r, c = torch.div(key, cols, rounding_mode="floor"), key % cols
    val = torch.rand(key.numel(), device=dev) / args.degree
    crow, col, val = graph_ops.coo_to_csr(r, c, val, rows, cols, assume_sorted=True)
    A = graph_ops.csr_tensor(crow, col, val, (rows, cols))
    nnz = int(val.numel())
    D, N = args.width, args.out_width
    H = torch.randn(cols, D, device=dev).to(torch.bfloat16)
    X = torch.randn(rows, D, device=dev).to(torch.bfloat16)
    W = (torch.randn(D, N, device=dev) / D**0.5).to(torch.bfloat16)
    peaks = load_measured_peaks()
    hbm, tflops = peaks.get("hbm_gbs", 6555.0) * 1e9, peaks.get("bf16_tflops", 1640.0) * 1e12

    res = {"ranks": p, "rows": rows, "nnz_per_rank": nnz, "width": D, "out_width": N, "kind": args.kind}

    # ---- SpMM + all-reduce
    def spmm_fused():
        return fused.spmm_all_reduce(A, H, group)

    def spmm_nccl():
        out = ops.spmm(A, H)
        dist.all_reduce(out, group=group)
        return out

    a = spmm_fused().float()
    b = spmm_nccl().float()
    res["spmm_max_rel_diff_fused_vs_nccl"] = ((a - b).abs().max() / b.abs().max()).item()
    res["spmm_fused_ms"] = timed(spmm_fused, args.warmup, args.iters)
    defaults = (fused.ONE_SHOT_MAX_RANKS, fused.TWO_SHOT, fused.SEGMENT_REDUCE, fused.SEGMENT_CHUNKS,
                fused.SEGMENT_BLOCKS)

    def each_form(prefix, fn):
        forms = [("one_shot", (p, False, False, 1, 64)), ("two_shot", (1, True, False, 1, 64)),
                 ("segment", (1, False, True, defaults[3], defaults[4]))]
        wanted = [f for f in args.forms.split(",") if f and f != "none"]
        forms = [f for f in forms if f[0] in wanted]
        if args.segment_sweep and "segment" in wanted:
            forms += [(f"segment_c{c}_b{b}", (1, False, True, c, b)) for c, b in
                      ((1, 64), (1, 148), (1, 296), (2, 64), (4, 32), (4, 148), (8, 64))]
        for name, cfg in forms:
            (fused.ONE_SHOT_MAX_RANKS, fused.TWO_SHOT, fused.SEGMENT_REDUCE, fused.SEGMENT_CHUNKS,
             fused.SEGMENT_BLOCKS) = cfg
            if name.startswith("segment"):
                got = fn().float()
                res[f"{prefix}_{name}_max_rel_diff_vs_nccl"] = ((got - b).abs().max() / b.abs().max()).item()
            res[f"{prefix}_{name}_ms"] = timed(fn, args.warmup, args.iters)
        (fused.ONE_SHOT_MAX_RANKS, fused.TWO_SHOT, fused.SEGMENT_REDUCE, fused.SEGMENT_CHUNKS,
         fused.SEGMENT_BLOCKS) = defaults

    each_form("spmm", spmm_fused)
    res["spmm_nccl_ms"] = timed(spmm_nccl, args.warmup, args.iters)
    res["spmm_only_ms"] = timed(lambda: ops.spmm(A, H), args.warmup, args.iters)
    msg = rows * D * 2
    link_s = 2 * (p - 1) / p * msg / (NVLINK_GBS * 1e9)
    flop_s = 2.0 * nnz * D / tflops
    gather_s = (nnz * (D * 2 + 8) + rows * D * 2) / hbm
    res["spmm_roofline_ms"] = max(link_s, flop_s) * 1e3
    res["spmm_hbm_gather_bound_ms"] = gather_s * 1e3
    res["spmm_fused_fraction_of_roofline"] = max(link_s, flop_s, gather_s) * 1e3 / res["spmm_fused_ms"]
    res["spmm_exposed_comm_ms"] = res["spmm_fused_ms"] - res["spmm_only_ms"]

    # ---- GEMM + all-reduce
    def gemm_fused():
        return fused.gemm_all_reduce(X, W, group, relu=True)

    def gemm_nccl():
        out = ops.gemm(X, W)
        dist.all_reduce(out, group=group)
        return torch.relu_(out)

    a = gemm_fused().float()
    b = gemm_nccl().float()
    res["gemm_max_rel_diff_fused_vs_nccl"] = ((a - b).abs().max() / b.abs().max()).item()
    res["gemm_fused_ms"] = timed(gemm_fused, args.warmup, args.iters)
    each_form("gemm", gemm_fused)
    res["gemm_nccl_ms"] = timed(gemm_nccl, args.warmup, args.iters)
    res["gemm_only_ms"] = timed(lambda: ops.gemm(X, W), args.warmup, args.iters)
    msg = rows * N * 2
    link_s = 2 * (p - 1) / p * msg / (NVLINK_GBS * 1e9)
    flop_s = 2.0 * rows * D * N / tflops
    hbm_s = (rows * D * 2 + rows * N * 2) / hbm
    res["gemm_roofline_ms"] = max(link_s, flop_s) * 1e3
    res["gemm_hbm_bound_ms"] = hbm_s * 1e3
    res["gemm_fused_fraction_of_roofline"] = max(link_s, flop_s, hbm_s) * 1e3 / res["gemm_fused_ms"]
    res["gemm_exposed_comm_ms"] = res["gemm_fused_ms"] - res["gemm_only_ms"]

    # ---- what the reference executes (fp32 libraries + NCCL)
    if not args.skip_reference:
        A64 = torch.sparse_csr_tensor(A.crow_indices().long(), A.col_indices().long(), A.values(), size=A.shape)
        Hf, Xf, Wf = H.float(), X.float(), W.float()

        def ref_spmm():
            out = torch.sparse.mm(A64, Hf)
            dist.all_reduce(out, group=group)
            return out

        def ref_gemm():
            out = torch.mm(Xf, Wf)
            dist.all_reduce(out, group=group)
            return torch.relu_(out)

        res["spmm_reference_ms"] = timed(ref_spmm, args.warmup, args.iters)
        res["gemm_reference_ms"] = timed(ref_gemm, args.warmup, args.iters)
    opc.check_status()
    from plexus_b200.parallel import symm

    res["multicast"] = bool(symm.axis_for(group).sym_mc)
    if rank == 0:
        print(json.dumps(res), flush=True)
    plx.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
