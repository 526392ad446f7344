"""SpMM micro-benchmark on one adjacency shard.

    python benchmarking/spmm.py <pt_file> <shard_row> <shard_col> <shard_x_col> [--iterations N --warmup W]
    python benchmarking/spmm.py --synthetic nodes,undirected_edges,width [--kind rmat|uniform]

Takes block (0, 0) of the adjacency split ``shard_row x shard_col`` ways and the matching
block of the features split ``shard_x_col`` ways (zero padded), prints the FLOP count
``2 * NNZ * D`` and times the product with CUDA events (reference:
benchmarking/spmm.py:12-125, which times ``torch.sparse.mm`` with a wall clock).  On a GPU
both this package's bf16 kernel and the cuSPARSE fp32 path of ``torch.sparse.mm`` are timed,
and the achieved fraction of the measured HBM bandwidth is reported for the former.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from plexus_b200 import ops  # noqa: E402
from plexus_b200.data import graph_ops  # noqa: E402
from plexus_b200.data.container import load_processed  # noqa: E402
from plexus_b200.parallel.sharding import pad_dimension  # noqa: E402
from plexus_b200.perf.comm_model import load_measured_peaks  # noqa: E402


def time_op(fn, warmup, iterations):
    for _ in range(warmup):
        fn()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iterations):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iterations / 1e3
    import time

    t0 = time.perf_counter()
    for _ in range(iterations):
        fn()
    return (time.perf_counter() - t0) / iterations


def shard00(edge_index, edge_weight, x, shard_row, shard_col, shard_x_col):
    n = x.shape[0]
    rows = pad_dimension(n, shard_row) // shard_row
    cols = pad_dimension(n, shard_col) // shard_col
    width = x.shape[1] if shard_x_col == 1 else pad_dimension(x.shape[1], shard_x_col) // shard_x_col
    r, c, v = graph_ops.extract_block(edge_index, edge_weight, 0, rows, 0, cols)
    crow, col, val = graph_ops.coo_to_csr(r, c, v, rows, cols)
    A = graph_ops.csr_tensor(crow, col, val, (rows, cols))
    xs = torch.zeros((cols, width), dtype=x.dtype, device=x.device)
    take_r, take_c = min(cols, n), min(width, x.shape[1])
    xs[:take_r, :take_c] = x[:take_r, :take_c]
    return A, xs


def multiply_sharded_matrices_padded(edge_index, edge_weight, x, shard_row, shard_col, shard_x_col,
                                     iterations, warmup_iterations, library=True):
    A, xs = shard00(edge_index, edge_weight, x, shard_row, shard_col, shard_x_col)
    nnz, D = A.values().numel(), xs.shape[1]
    print("Theoretical # of FLOPs (2 * NNZ * D): " + str(2 * nnz * D))
    results = {}
    if torch.cuda.is_available():
        dev = torch.device("cuda")
        Ad = A.to(dev)
        Dp = (D + 7) // 8 * 8
        Hb = torch.zeros((xs.shape[0], Dp), dtype=torch.bfloat16, device=dev)
        Hb[:, :D] = xs.to(dev)
        t = time_op(lambda: ops.spmm(Ad, Hb), warmup_iterations, iterations)
        moved = nnz * (Dp * 2 + 8) + A.shape[0] * (Dp * 2 + 4)
        peak = load_measured_peaks().get("hbm_gbs", 6555.0)
        results["plexus_b200 bf16"] = t
        print(f"plexus_b200 SpMM (bf16, fp32 acc): {t * 1e3:.3f} ms  "
              f"{2 * nnz * Dp / t / 1e12:.2f} TFLOP/s  gathered+written {moved / t / 1e9:.0f} GB/s "
              f"= {moved / t / 1e9 / peak:.2f} of measured HBM copy bandwidth")
        if library:
            A64 = torch.sparse_csr_tensor(Ad.crow_indices().long(), Ad.col_indices().long(), Ad.values(),
                                          size=Ad.shape)
            Hf = xs.to(dev, torch.float32)
            t = time_op(lambda: torch.sparse.mm(A64, Hf), warmup_iterations, iterations)
            results["torch.sparse.mm fp32"] = t
            print(f"torch.sparse.mm (cuSPARSE, fp32): {t * 1e3:.3f} ms")
    else:
        t = time_op(lambda: torch.sparse.mm(A, xs.float()), warmup_iterations, iterations)
        results["torch.sparse.mm cpu"] = t
    print(f"Average time per sparse matrix multiplication: {list(results.values())[0]:.6f} seconds")
    return results


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Multiply sharded sparse and dense tensors with padding.")
    parser.add_argument("pt_file", type=str, nargs="?", default=None,
                        help="Path to a processed .pt file containing the data")
    parser.add_argument("shard_row", type=int, nargs="?", default=1)
    parser.add_argument("shard_col", type=int, nargs="?", default=1)
    parser.add_argument("shard_x_col", type=int, nargs="?", default=1)
    parser.add_argument("--iterations", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--synthetic", type=str, default=None, help="nodes,undirected_edges,width")
    parser.add_argument("--kind", type=str, default="rmat")
    parser.add_argument("--no_library", action="store_true")
    args = parser.parse_args()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    if args.synthetic:
        from plexus_b200.data.synthetic import synthetic_graph

        n, e, d = (int(v) for v in args.synthetic.split(","))
        data, _ = synthetic_graph(n, e, d, 2, seed=0, kind=args.kind, device=dev, with_masks=False)
    else:
        data, _ = load_processed(args.pt_file)
        data = data.to(dev)
    multiply_sharded_matrices_padded(data.edge_index, data.edge_weight, data.x, args.shard_row,
                                     args.shard_col, args.shard_x_col, args.iterations, args.warmup,
                                     library=not args.no_library)
