"""Epoch time of one graph on several grid shapes, generating the graph once.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 benchmarking/grid_sweep.py \
        --nodes 233000 --edges 57400000 --features 602 --hidden 256 --classes 41 \
        --grids 8x1x1,1x8x1,1x1x8,2x2x2 [--comm fused|nccl] [--steps 5 --warmup 3]

Every grid re-initialises the process grid, cuts the shards out of the resident global edge list,
builds the model and times ``steps`` epochs (forward, loss, backward, AdamW over weights and
features) after ``warmup`` epochs: CUDA events on the GPU, max over ranks.  One JSON line per grid
with the measured epoch, the prediction of ``perf/epoch_model.py`` and its region breakdown, so the
model can be checked against a sweep; the last line ranks the grids.  ``--backend gloo`` runs the
same loop on CPU ranks (wall-clock times; for checking the tool, not for numbers).

The reference compares grid shapes by running its example once per shape by hand
(examples/run_4.sh) and its models separately (performance/*.py).
"""

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", type=int, default=2449029)
    ap.add_argument("--edges", type=int, default=60634000, help="undirected edges before symmetrisation")
    ap.add_argument("--features", type=int, default=100)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--classes", type=int, default=47)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--grids", type=str, required=True, help="comma-separated XxYxZ list")
    ap.add_argument("--comm", type=str, default="fused", choices=["fused", "nccl"])
    ap.add_argument("--backend", type=str, default=None, choices=["nccl", "gloo"])
    ap.add_argument("--dtype", type=str, default=None, choices=["bf16", "fp32"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)

    use_cuda = torch.cuda.is_available() and args.backend != "gloo"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(args.backend or ("nccl" if use_cuda else "gloo"))
    rank = dist.get_rank() if dist.is_initialized() else 0

    import plexus_b200 as plx
    from plexus_b200.data.synthetic import synthetic_graph
    from plexus_b200.models.cross_entropy import parallel_cross_entropy
    from plexus_b200.models.net import Net
    from plexus_b200.optim import FusedAdamW
    from plexus_b200.perf.epoch_model import predict_epoch_ms
    from plexus_b200.utils.dataloader import DataLoader
    from plexus_b200.utils.dataset import preprocess_data
    from plexus_b200.utils.general import set_seed

    set_seed(args.seed)
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    raw, nc = synthetic_graph(args.nodes, args.edges, args.features, args.classes, seed=args.seed, kind="rmat",
                              device=device)
    data, _ = preprocess_data(raw, nc, double_perm=True, normalized=True, seed=args.seed)
    del raw
    nnz = int(data.edge_index.shape[1])
    dims = [args.features] + [args.hidden] * (args.layers - 1) + [args.classes]
    dtype = {"bf16": torch.bfloat16, "fp32": torch.float32, None: None}[args.dtype]

    results = []
    for spec in args.grids.split(","):
        grid = tuple(int(v) for v in spec.lower().split("x"))
        if grid[0] * grid[1] * grid[2] != world:
            raise SystemExit(f"grid {spec} does not use {world} ranks")
        plx.init(*grid, comm=args.comm if (use_cuda and world > 1) else "nccl", dtype=dtype,
                 device=None if use_cuda else "cpu")
        from plexus_b200.parallel import fused

        forms_before = dict(fused.op_counts)
        adj, feats, labels, N, F, C = DataLoader(None, args.layers, data=(data, nc)).load()
        model = Net(args.layers, F, args.hidden, C, seed=args.seed)
        opt = FusedAdamW(list(model.parameters()) + [feats], lr=3e-3)

        def step():
            opt.zero_grad(set_to_none=True)
            loss = parallel_cross_entropy(model(feats, adj), labels, args.layers, N, C)
            loss.backward()
            opt.step()
            return loss

        for _ in range(args.warmup):
            step()
        if dist.is_initialized():
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            loss = step()
        if use_cuda:
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
        else:
            ms = (time.perf_counter() - t0) * 1e3 / args.steps
        if dist.is_initialized():
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        model_ms = predict_epoch_ms(grid, args.nodes, nnz, dims)
        rec = {"grid": list(grid), "epoch_ms": round(ms, 3), "model_ms": round(model_ms["total"], 3),
               "model_regions": {k: round(v, 3) for k, v in model_ms.items() if k != "total"},
               "loss": float(loss.detach()), "comm": args.comm if world > 1 else "none", "nnz": nnz,
               # how the matrix collectives were carried (library = NCCL after the compute kernel)
               "collective_forms": {k: v - forms_before.get(k, 0) for k, v in fused.op_counts.items()
                                    if v - forms_before.get(k, 0)}}
        results.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)
        del adj, feats, labels, model, opt
        plx.shutdown()
        if use_cuda:
            torch.cuda.empty_cache()
    if rank == 0:
        order = sorted(results, key=lambda r: r["epoch_ms"])
        print(json.dumps({"ranking": [r["grid"] for r in order], "epoch_ms": [r["epoch_ms"] for r in order]}),
              flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
