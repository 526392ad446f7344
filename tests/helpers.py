"""Shared test helpers: small graphs, serial oracle, multi-process launcher."""

import os
import sys
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def small_processed_graph(n=96, e=400, f=10, c=5, seed=3, double_perm=True, kind="rmat", unlabeled=0.1):
    from plexus_b200.data.synthetic import synthetic_graph
    from plexus_b200.utils.dataset import preprocess_data

    raw, _ = synthetic_graph(n, e, f, c, seed=seed, kind=kind)
    if unlabeled:
        drop = torch.rand(n, generator=torch.Generator().manual_seed(seed)) < unlabeled
        raw.y = torch.where(drop, torch.full_like(raw.y, -1), raw.y)
    return preprocess_data(raw, c, double_perm=double_perm, normalized=True, seed=seed)


def dense_adj(ei, ew, n):
    A = torch.zeros(n, n, dtype=torch.float64)
    A.index_put_((ei[0], ei[1]), ew.double(), accumulate=True)
    return A


def oracle(data, num_classes, num_layers, hidden, seed, dtype=torch.float64):
    """Serial dense run: returns (loss, weight grads list, feature grad, logits)."""
    from plexus_b200.models.gcn_conv import init_full_weight

    n = data.x.shape[0]
    adjs = [dense_adj(data.edge_index, data.edge_weight, n)]
    if hasattr(data, "edge_index_2"):
        adjs.append(dense_adj(data.edge_index_2, data.edge_weight_2, n))
    dims = [data.x.shape[1]] + [hidden] * (num_layers - 1) + [num_classes]
    ws = [init_full_weight(dims[i], dims[i + 1], i, seed).to(dtype).requires_grad_() for i in range(num_layers)]
    x = data.x.to(dtype).clone().requires_grad_()
    h = x
    for l, w in enumerate(ws):
        h = adjs[l % len(adjs)] @ h @ w
        if l != num_layers - 1:
            h = torch.relu(h)
    y = data.y_2 if (hasattr(data, "y_2") and num_layers % 2 == 0) else data.y
    loss = torch.nn.functional.cross_entropy(h, y, ignore_index=-1, reduction="sum") / n
    loss.backward()
    return loss.detach(), [w.grad for w in ws], x.grad, h.detach()


def _entry(rank, world, fn, init_file, args, errq):
    try:
        os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), str(world)
        dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
        torch.set_num_threads(1)
        fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


_ctx = None


def _context():
    """Fork-server start method with torch preloaded: every rank is forked from one clean server
    process that imported torch once, instead of paying the interpreter + ``import torch`` start-up
    (several seconds here) per rank as ``spawn`` does.  CPU tests only; GPU tests spawn."""
    global _ctx
    if _ctx is None:
        _ctx = mp.get_context("forkserver")
        _ctx.set_forkserver_preload(["torch", "torch.distributed", "numpy"])
    return _ctx


def run_distributed(fn, world, *args, timeout=240):
    """Run ``fn(rank, world, *args)`` in ``world`` gloo processes; raise on any failure."""
    ctx = _context()
    errq = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "init")
        procs = [ctx.Process(target=_entry, args=(r, world, fn, init_file, args, errq)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        alive = [p for p in procs if p.is_alive()]
        for p in alive:
            p.terminate()
        errs = []
        while not errq.empty():
            errs.append(errq.get())
        if errs:
            raise AssertionError("\n".join(f"[rank {r}]\n{tb}" for r, tb in errs))
        assert not alive, "distributed test timed out"
        bad = [p.exitcode for p in procs if p.exitcode != 0]
        assert not bad, f"worker exit codes {bad}"
