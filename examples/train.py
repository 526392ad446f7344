"""Train a 3D-parallel GCN on a preprocessed (or synthetic) graph.

Launch one process per GPU, e.g.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/train.py \
        --data_dir <dir> --G_intra_r 2 --G_intra_c 2 --G_intra_d 2 --num_epochs 10

The flags of the reference's example are kept (reference:
examples/train.py:19-52); added: ``--grid auto`` (ask the cost models),
``--synthetic`` (seeded R-MAT graph instead of files), ``--dtype``, ``--comm``,
``--checkpoint_dir`` / ``--resume`` / ``--checkpoint_every``,
``--metrics_file``, ``--eval`` (train/val/test accuracy from the masks),
``--epoch_timeout`` (watchdog) and ``--backend``.
"""

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import plexus_b200 as plx  # noqa: E402
from plexus_b200.models.cross_entropy import parallel_accuracy, parallel_cross_entropy  # noqa: E402
from plexus_b200.models.net import Net  # noqa: E402
from plexus_b200.optim import FusedAdamW  # noqa: E402
from plexus_b200.parallel.watchdog import EpochWatchdog, Heartbeat  # noqa: E402
from plexus_b200.utils import checkpoint as ckpt  # noqa: E402
from plexus_b200.utils.dataloader import DataLoader  # noqa: E402
from plexus_b200.utils.general import print_axonn_timer_data, set_seed  # noqa: E402
from plexus_b200.parallel import collectives as coll  # noqa: E402
from plexus_b200.perf.epoch_model import predict_epoch_ms  # noqa: E402
from plexus_b200.utils.metrics import MetricsSink, max_over_ranks, peak_memory_gb, shard_nnz_imbalance  # noqa: E402
from plexus_b200.utils.timers import get_timers  # noqa: E402


def create_parser():
    parser = argparse.ArgumentParser()
    parser.add_argument("--data_dir", type=str)
    parser.add_argument("--G_intra_r", type=int, default=1)
    parser.add_argument("--G_intra_c", type=int, default=1)
    parser.add_argument("--G_intra_d", type=int, default=1)
    parser.add_argument("--gpus_per_node", type=int, default=None)
    parser.add_argument("--num_epochs", type=int, default=2)
    parser.add_argument("--block_aggregation", action="store_true", default=False,
                        help="Enable 1D blocking in aggregation")
    parser.add_argument("--overlap_aggregation", action="store_true", default=False,
                        help="Enable overlap in aggregation")
    parser.add_argument("--tune_gemms", action="store_true", default=False,
                        help="Enables tuning of dense matrix multiplications")
    parser.add_argument("--timing_start_epoch", type=int, default=None)
    parser.add_argument("--timing_end_epoch", type=int, default=None)
    parser.add_argument("--lr", type=float, default=3e-3)
    parser.add_argument("--weight_decay", type=float, default=0.0)
    parser.add_argument("--num_gcn_layers", type=int, default=3)
    parser.add_argument("--hidden_size", type=int, default=128)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--dropout", type=float, default=0.0,
                        help="dropout probability on the hidden activations (0 = the reference model)")
    # additions
    parser.add_argument("--grid", type=str, default=None, help="'auto' or 'XxYxZ'")
    parser.add_argument("--backend", type=str, default=None, help="nccl (GPU) or gloo (CPU)")
    parser.add_argument("--comm", type=str, default=None, choices=["nccl", "fused"])
    parser.add_argument("--dtype", type=str, default=None, choices=["bf16", "fp32"])
    parser.add_argument("--synthetic", type=str, default=None,
                        help="nodes,undirected_edges,features,classes[,kind] instead of --data_dir")
    parser.add_argument("--sharded_synthetic", action="store_true", default=False,
                        help="with --synthetic: every rank generates only its own shards (the edge count "
                             "is then the number of raw generator edges before de-duplication); for graphs "
                             "whose global edge list does not fit one device")
    parser.add_argument("--single_perm", action="store_true", default=False)
    parser.add_argument("--checkpoint_dir", type=str, default=None)
    parser.add_argument("--checkpoint_every", type=int, default=0)
    parser.add_argument("--resume", action="store_true", default=False)
    parser.add_argument("--consolidated", type=str, default=None,
                        help="path of a grid-independent checkpoint to load / write at the end")
    parser.add_argument("--metrics_file", type=str, default=None)
    parser.add_argument("--eval", action="store_true", default=False)
    parser.add_argument("--train_mask_only", action="store_true", default=False)
    parser.add_argument("--epoch_timeout", type=float, default=0.0)
    return parser


def train(model, optimizer, features_local, adj_shards, labels, num_nodes, num_classes, row_weight=None):
    """One epoch: zero_grad / forward / loss / backward / step on the whole graph."""
    model.train()
    optimizer.zero_grad(set_to_none=True)
    output = model(features_local, adj_shards)
    loss = parallel_cross_entropy(output, labels, model.num_gcn_layers, num_nodes, num_classes, row_weight)
    loss.backward()
    optimizer.step()
    return loss, output


def _parse_injection(spec):
    """``rank:epoch[:kind]`` with kind ``exit`` (default), ``raise``, ``stall`` or ``status``; None if unset.

    ``status`` fakes, on the host, what a kernel leaves behind when one of its bounded waits gives
    up: a TIMEOUT record in the status words, which the check after the step must turn into an error."""
    if not spec:
        return None
    parts = spec.split(":")
    kind = parts[2] if len(parts) > 2 else "exit"
    if kind not in ("exit", "raise", "stall", "status"):
        raise SystemExit("PLEXUS_INJECT_FAILURE kind must be exit, raise, stall or status")
    return int(parts[0]), int(parts[1]), kind


def _parse_grid(args, world):
    if args.grid and args.grid != "auto":
        x, y, z = (int(v) for v in args.grid.lower().split("x"))
        return x, y, z
    if args.grid == "auto":
        return None
    return args.G_intra_r, args.G_intra_c, args.G_intra_d


def main(argv=None):
    args = create_parser().parse_args(argv)
    set_seed(args.seed)
    use_cuda = torch.cuda.is_available() and args.backend != "gloo"
    backend = args.backend or ("nccl" if use_cuda else "gloo")
    if "RANK" in os.environ:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group(backend=backend)
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0

    synthetic = None
    if args.synthetic:
        parts = args.synthetic.split(",")
        n, e, f, c = (int(v) for v in parts[:4])
        kind = parts[4] if len(parts) > 4 else "rmat"
        synthetic = (n, e, f, c, kind)

    grid = _parse_grid(args, world)
    if grid is None:
        if synthetic is None:
            meta = os.path.join(args.data_dir, "metadata.pt")
            if not os.path.exists(meta):
                raise SystemExit("--grid auto needs a partitioned data_dir (metadata.pt) or --synthetic")
            n, f, c = torch.load(meta, weights_only=False)
            e = n * 25
        dims = [f] + [args.hidden_size] * (args.num_gcn_layers - 1) + [c]
        grid = plx.choose_grid(world, n, 2 * e + n, dims)
        if rank == 0:
            print(f"cost models chose grid X{grid[0]} Y{grid[1]} Z{grid[2]}")

    plx.init(
        G_intra_r=grid[0], G_intra_c=grid[1], G_intra_d=grid[2],
        gpus_per_node=args.gpus_per_node,
        enable_internal_timers=True,
        block_aggregation=args.block_aggregation,
        overlap_aggregation=args.overlap_aggregation,
        tune_gemms=args.tune_gemms,
        comm=args.comm,
        dtype={"bf16": torch.bfloat16, "fp32": torch.float32, None: None}[args.dtype],
        device=None if use_cuda else "cpu",
    )

    if synthetic is not None and args.sharded_synthetic:
        from plexus_b200.data.sharded_synthetic import ShardedSyntheticGraph

        n, e, f, c, kind = synthetic
        dev = torch.device("cuda", torch.cuda.current_device()) if use_cuda else "cpu"
        loader = DataLoader(None, args.num_gcn_layers,
                            source=ShardedSyntheticGraph(n, e, f, c, seed=args.seed, kind=kind, device=dev))
    elif synthetic is not None:
        from plexus_b200.data.synthetic import synthetic_graph
        from plexus_b200.utils.dataset import preprocess_data

        n, e, f, c, kind = synthetic
        dev = "cuda" if use_cuda else "cpu"
        raw, _ = synthetic_graph(n, e, f, c, seed=args.seed, kind=kind, device=dev)
        data = preprocess_data(raw, c, double_perm=not args.single_perm, normalized=True, seed=args.seed)
        del raw
        loader = DataLoader(None, args.num_gcn_layers, data=data)
    else:
        loader = DataLoader(args.data_dir, args.num_gcn_layers)
    adj_shards, features, labels, num_nodes, num_features, num_classes = loader.load()

    model = Net(args.num_gcn_layers, num_features, args.hidden_size, num_classes, seed=args.seed,
                dropout=args.dropout)
    optimizer = FusedAdamW(list(model.parameters()) + [features], lr=args.lr, weight_decay=args.weight_decay)

    start_epoch = 0
    if args.resume:
        import json

        meta = os.path.join(args.checkpoint_dir, "meta.json") if args.checkpoint_dir else None
        same_grid = False
        if meta and os.path.exists(meta):
            with open(meta) as f:
                same_grid = tuple(json.load(f)["grid"]) == tuple(grid)
        if same_grid:
            start_epoch = ckpt.load_sharded(args.checkpoint_dir, model, optimizer, features)
        elif args.consolidated and os.path.exists(args.consolidated):
            # a different grid (or no sharded checkpoint): re-shard the grid-independent form
            start_epoch = ckpt.load_consolidated(args.consolidated, model, optimizer, features)
            if rank == 0:
                print(f"resumed from the consolidated checkpoint at epoch {start_epoch} on grid {tuple(grid)}")
        elif meta and os.path.exists(meta):
            raise SystemExit("the sharded checkpoint was written on another grid; pass --consolidated FILE "
                             "(saved with --checkpoint_every) to resume on this one")

    sink = MetricsSink(args.metrics_file)
    # global nonzeros: the layer-0 blocks tile the matrix once per inner-axis replica
    nnz = torch.tensor([float(adj_shards[0][0].values().numel())], dtype=torch.float64,
                       device=adj_shards[0][0].values().device)
    if dist.is_initialized() and world > 1:
        dist.all_reduce(nnz)
    total_nnz = int(nnz.item()) // max(1, grid[1])
    dims = [num_features] + [args.hidden_size] * (args.num_gcn_layers - 1) + [num_classes]
    model_ms = predict_epoch_ms(grid, num_nodes, total_nnz, dims)
    sink.log(event="start", grid=list(grid), world=world, num_nodes=num_nodes, num_features=num_features,
             num_classes=num_classes, nnz=total_nnz, nnz_imbalance=shard_nnz_imbalance(adj_shards),
             model_epoch_ms={k: round(v, 3) for k, v in model_ms.items()})
    row_weight = None
    if args.train_mask_only and "train_mask" in loader.masks:
        row_weight = loader.masks["train_mask"].to(torch.float32)

    watchdog = EpochWatchdog(args.epoch_timeout) if args.epoch_timeout > 0 else None
    heartbeat = None
    if dist.is_initialized() and world > 1:
        try:
            heartbeat = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world)
        except Exception:
            heartbeat = None

    if dist.is_initialized():
        dist.barrier()
    t0 = args.timing_start_epoch if args.timing_start_epoch is not None else 0
    t1 = args.timing_end_epoch if args.timing_end_epoch is not None else args.num_epochs - 1
    timers = get_timers()
    inject = _parse_injection(os.environ.get("PLEXUS_INJECT_FAILURE"))
    for i in range(start_epoch, args.num_epochs):
        if inject is not None and inject[0] == rank and inject[1] == i:
            # host-side fault injection, between steps: no kernel or collective of this rank is in flight
            if heartbeat is not None and inject[2] == "exit":
                heartbeat.announce_exit("injected failure")
            if inject[2] == "exit":
                print(f"[rank {rank}] injected failure: exiting before epoch {i}", flush=True)
                os._exit(3)
            if inject[2] == "raise":
                raise RuntimeError(f"injected failure on rank {rank} before epoch {i}")
            if inject[2] == "status":
                plx.runtime.inject_status_timeout()
            if inject[2] == "stall":
                import time as _time

                print(f"[rank {rank}] injected failure: stalling before epoch {i}", flush=True)
                _time.sleep(10 ** 6)
        if heartbeat is not None:
            heartbeat.beat(i)
            heartbeat.check_peers(max_age_s=max(60.0, 4 * args.epoch_timeout))
        if watchdog is not None:
            watchdog.begin(i)
        timed = t0 <= i <= t1
        if use_cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        if timed:
            timers.start("epoch " + str(i))
        loss, output = train(model, optimizer, features, adj_shards, labels, num_nodes, num_classes, row_weight)
        if timed:
            timers.stop("epoch " + str(i))
        if use_cuda:
            ev1.record()
        if timed:
            times, _counts = timers.get_times()
            print_axonn_timer_data(times)
        loss_val = float(loss)
        if watchdog is not None:
            watchdog.end()
        # a kernel whose bounded wait gave up returned without its result: stop here, before the
        # loss is reported as valid and before a checkpoint could persist the damaged state (the
        # supervisor then restarts from the last good checkpoint)
        plx.check_status()
        if rank == 0:
            print("Epoch: {:03d}, Train Loss: {:.4f}".format(i, loss_val))
        rec = dict(event="epoch", epoch=i, loss=loss_val, peak_mem_gb=peak_memory_gb(),
                   collective_bytes=coll.bytes_moved(reset=True))
        if use_cuda:
            torch.cuda.synchronize()
            rec["epoch_ms_max"] = max_over_ranks(ev0.elapsed_time(ev1))
            # measured epoch against the per-region model of this machine (1.0 = as modelled)
            rec["model_over_measured"] = round(model_ms["total"] / max(rec["epoch_ms_max"], 1e-9), 3)
        if args.eval:
            for m in ("train_mask", "val_mask", "test_mask"):
                if m in loader.masks:
                    rec["acc_" + m[:-5]] = parallel_accuracy(
                        output, labels, args.num_gcn_layers, num_nodes, num_classes, loader.masks[m])
            if rank == 0:
                print("  " + ", ".join(f"{k}: {v:.4f}" for k, v in rec.items() if k.startswith("acc_")))
        sink.log(**rec)
        if args.checkpoint_every and (i + 1) % args.checkpoint_every == 0:
            if args.checkpoint_dir:
                ckpt.save_sharded(args.checkpoint_dir, model, optimizer, features, i)
            if args.consolidated:
                # grid-independent copy as well, so a restart may use fewer or more GPUs
                ckpt.save_consolidated(args.consolidated, model, optimizer, features, num_nodes, num_features,
                                       epoch=i)
    if args.consolidated:
        ckpt.save_consolidated(args.consolidated, model, optimizer, features, num_nodes, num_features,
                               epoch=args.num_epochs - 1)
    if watchdog is not None:
        watchdog.close()
    sink.close()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
