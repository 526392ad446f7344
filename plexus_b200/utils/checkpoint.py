"""Checkpoint / resume.

Two on-disk forms:

* **sharded** (``<dir>/step_<epoch>/rank{r}.pt`` + ``<dir>/meta.json``): each rank
  writes its own model ``state_dict`` (keys ``layers.{l}.weight``), optimizer
  state, feature shard, RNG state and epoch.  Files are written to a temporary
  name and renamed, every save goes to its own sub-directory, and ``meta.json``
  (replaced atomically after all ranks finished) names the sub-directory of
  the last complete save - so a crash at any point of a save leaves the
  previous checkpoint intact and consistent.  Resuming needs the same grid.
* **consolidated** (one file): the full unpadded weight matrices ``W_l``, the
  full feature matrix and, optionally, the Adam moments in the same full
  layout.  It does not depend on the grid, so a run can resume on a different
  ``(X, Y, Z)``: every rank cuts its shard out of the full matrices on load.

The reference has no checkpointing (its example keeps the layers in a plain
list, so even ``state_dict()`` is empty; reference: examples/train.py:65).
"""

from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..parallel.grid import get_grid
from ..parallel.sharding import depth_slice, pad_dimension, shard_2d


class CheckpointError(RuntimeError):
    pass


def _atomic_torch_save(obj, path: str) -> None:
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(obj, tmp)
    with open(tmp, "rb") as f:
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


# ------------------------------------------------------------------ sharded
def _step_dir(epoch: int) -> str:
    return f"step_{int(epoch):08d}"


def save_sharded(ckpt_dir: str, model, optimizer, features, epoch: int, extra: Optional[dict] = None,
                 keep: int = 2):
    """Write one checkpoint as ``<dir>/step_<epoch>/rank{r}.pt`` and publish it in ``meta.json``.

    A checkpoint becomes visible only when ``meta.json`` is replaced (atomically, by rank 0,
    after every rank has finished its file), and the files of the previously published
    checkpoint are never touched by a later save: a rank that dies while saving leaves the old
    ``meta.json`` pointing at a complete, consistent set of rank files.  The last ``keep``
    published checkpoints are kept on disk.
    """
    import shutil

    rank, world = _world()
    g = get_grid()
    sub = _step_dir(epoch)
    os.makedirs(os.path.join(ckpt_dir, sub), exist_ok=True)
    state = {
        "model": {k: v.detach().cpu() for k, v in model.state_dict().items()},
        "optimizer": optimizer.state_dict() if optimizer is not None else None,
        "features": features.detach().cpu() if features is not None else None,
        "epoch": epoch,
        "rng": {
            "python": random.getstate(),
            "numpy": np.random.get_state(),
            "torch": torch.get_rng_state(),
        },
        "grid": (g.X, g.Y, g.Z),
        "rank": rank,
    }
    _atomic_torch_save(state, os.path.join(ckpt_dir, sub, f"rank{rank}.pt"))
    _barrier()
    if rank == 0:
        meta = {"grid": [g.X, g.Y, g.Z], "world_size": world, "epoch": epoch, "format": 2, "dir": sub}
        meta.update(extra or {})
        tmp = os.path.join(ckpt_dir, "meta.json.tmp")
        with open(tmp, "w") as f:
            json.dump(meta, f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, os.path.join(ckpt_dir, "meta.json"))
        # drop checkpoints older than the last `keep` (the one just published included)
        steps = sorted(d for d in os.listdir(ckpt_dir) if d.startswith("step_") and d <= sub)
        for d in steps[: max(0, len(steps) - max(1, keep))]:
            shutil.rmtree(os.path.join(ckpt_dir, d), ignore_errors=True)
    _barrier()


def load_sharded(ckpt_dir: str, model, optimizer, features) -> int:
    """Restore this rank's shard; returns the epoch to resume from.

    Raises :class:`CheckpointError` if the rank file does not belong to the published checkpoint
    (other epoch or grid than ``meta.json`` states) or if the ranks would resume from different
    epochs.
    """
    rank, world = _world()
    g = get_grid()
    meta_path = os.path.join(ckpt_dir, "meta.json")
    if not os.path.exists(meta_path):
        raise CheckpointError(f"no complete checkpoint in {ckpt_dir} (meta.json missing)")
    with open(meta_path) as f:
        meta = json.load(f)
    if tuple(meta["grid"]) != (g.X, g.Y, g.Z):
        raise CheckpointError(
            f"sharded checkpoint was written on grid {meta['grid']}, current grid is "
            f"{[g.X, g.Y, g.Z]}; use the consolidated form to change the grid"
        )
    # format 1 kept the rank files next to meta.json
    path = os.path.join(ckpt_dir, meta.get("dir", ""), f"rank{rank}.pt")
    try:
        state = torch.load(path, weights_only=False, map_location="cpu")
    except Exception as e:
        raise CheckpointError(f"cannot read {path}: {e}") from e
    if int(state["epoch"]) != int(meta["epoch"]) or tuple(state["grid"]) != tuple(meta["grid"]):
        raise CheckpointError(
            f"{path} holds epoch {state['epoch']} on grid {list(state['grid'])}, but meta.json publishes "
            f"epoch {meta['epoch']} on grid {meta['grid']}: the checkpoint is inconsistent")
    if world > 1:
        # every rank must resume from the same epoch, or their collective sequences diverge
        dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
        lo_hi = torch.tensor([-int(state["epoch"]), int(state["epoch"])], dtype=torch.int64, device=dev)
        dist.all_reduce(lo_hi, op=dist.ReduceOp.MAX)
        if -int(lo_hi[0]) != int(lo_hi[1]):
            raise CheckpointError(f"ranks hold checkpoints of different epochs ({-int(lo_hi[0])} .. {int(lo_hi[1])})")
    model.load_state_dict(state["model"])
    if optimizer is not None and state["optimizer"] is not None:
        optimizer.load_state_dict(state["optimizer"])
    if features is not None and state["features"] is not None:
        with torch.no_grad():
            features.copy_(state["features"].to(features.device, features.dtype))
    random.setstate(state["rng"]["python"])
    np.random.set_state(state["rng"]["numpy"])
    torch.set_rng_state(state["rng"]["torch"])
    return int(state["epoch"]) + 1


# ------------------------------------------------------------- consolidated
def _gather_objects(obj):
    rank, world = _world()
    if world == 1:
        return [obj]
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


def _weight_piece(layer, flat: torch.Tensor):
    return {
        "inner": layer.inner_rank, "outer": layer.w_col_rank, "depth": layer.depth_rank,
        "sharded": layer.gather_weights, "flat": flat.detach().float().cpu(),
    }


def _assemble_weight(layer, pieces) -> torch.Tensor:
    """Full unpadded ``[in, out]`` matrix from every rank's flat piece."""
    li, lo = layer.local_in_channels, layer.local_weight_cols
    full = torch.zeros(layer.in_channels, layer.out_channels)
    d = layer.depth_group_size if layer.gather_weights else 1
    n = li * lo // d
    blocks: Dict[tuple, torch.Tensor] = {}
    for p in pieces:
        key = (p["inner"], p["outer"])
        blk = blocks.setdefault(key, torch.zeros(li * lo))
        if p["sharded"]:
            blk[p["depth"] * n : (p["depth"] + 1) * n] = p["flat"]
        else:
            blk.copy_(p["flat"])
    for (i, o), blk in blocks.items():
        full[i * li : (i + 1) * li, o * lo : (o + 1) * lo] = blk.view(li, lo)
    return full[: layer.true_in_channels, : layer.true_out_channels].clone()


def _cut_weight(layer, full: torch.Tensor) -> torch.Tensor:
    padded = torch.nn.functional.pad(
        full, (0, layer.out_channels - full.shape[1], 0, layer.in_channels - full.shape[0])
    )
    blk = shard_2d(padded, layer.inner_group_size, layer.inner_rank, layer.w_col_parts, layer.w_col_rank)
    flat = blk.contiguous().reshape(-1)
    if layer.gather_weights:
        flat = depth_slice(flat, layer.depth_group_size, layer.depth_rank)
    return flat.clone()


def _feature_layout(num_nodes: int, num_features: int, flat_len: int):
    g = get_grid()
    rows = pad_dimension(num_nodes, g.X) // g.X
    cols = (flat_len * g.Z) // rows if rows else 0
    return g, rows, cols


def _assemble_features(pieces, num_nodes, num_features) -> torch.Tensor:
    g = get_grid()
    any_len = pieces[0]["flat"].numel()
    _, rows, cols = _feature_layout(num_nodes, num_features, any_len)
    full = torch.zeros(rows * g.X, cols * g.Y)
    blocks: Dict[tuple, torch.Tensor] = {}
    for p in pieces:
        blk = blocks.setdefault((p["x"], p["y"]), torch.zeros(any_len * g.Z))
        blk[p["z"] * any_len : (p["z"] + 1) * any_len] = p["flat"]
    for (x, y), blk in blocks.items():
        full[x * rows : (x + 1) * rows, y * cols : (y + 1) * cols] = blk[: rows * cols].view(rows, cols)
    return full[:num_nodes, :num_features].clone()


def _cut_features(full: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    g = get_grid()
    n = like.numel()
    N, Fd = full.shape
    _, rows, cols = _feature_layout(N, Fd, n)
    padded = torch.nn.functional.pad(full, (0, cols * g.Y - Fd, 0, rows * g.X - N))
    blk = padded[g.coord("x") * rows : (g.coord("x") + 1) * rows, g.coord("y") * cols : (g.coord("y") + 1) * cols]
    flat = torch.nn.functional.pad(blk.contiguous().reshape(-1), (0, n * g.Z - rows * cols))
    return flat[g.coord("z") * n : (g.coord("z") + 1) * n].clone()


def _opt_state_of(optimizer, p):
    st = optimizer.state.get(p, None) if optimizer is not None else None
    return st if st else None


def save_consolidated(path: str, model, optimizer=None, features=None, num_nodes: int = 0,
                      num_features: int = 0, epoch: int = 0, extra: Optional[dict] = None) -> None:
    """Gather the full matrices on rank 0 and write one grid-independent file."""
    rank, _ = _world()
    g = get_grid()
    out = {"weights": [], "epoch": epoch, "format": 1, "extra": extra or {}}
    moments = {"exp_avg": [], "exp_avg_sq": []}
    step = 0
    for layer in model.layers:
        pieces = _gather_objects(_weight_piece(layer, layer.weight))
        out["weights"].append(_assemble_weight(layer, pieces) if rank == 0 else None)
        st = _opt_state_of(optimizer, layer.weight)
        for k in moments:
            have = _gather_objects(_weight_piece(layer, st[k]) if st else None)
            moments[k].append(
                _assemble_weight(layer, have) if (rank == 0 and all(h is not None for h in have)) else None
            )
        if st:
            step = int(st["step"])
    if features is not None:
        x, y, z = g.coords
        st = _opt_state_of(optimizer, features)
        src = st["master"] if (st and st.get("master") is not None) else features

        def piece(t):
            return {"x": x, "y": y, "z": z, "flat": t.detach().float().cpu()}

        pieces = _gather_objects(piece(src))
        out["features"] = _assemble_features(pieces, num_nodes, num_features) if rank == 0 else None
        for k in moments:
            have = _gather_objects(piece(st[k]) if st else None)
            out["features_" + k] = (
                _assemble_features(have, num_nodes, num_features)
                if (rank == 0 and all(h is not None for h in have)) else None
            )
    out["moments"] = moments
    out["step"] = step
    if rank == 0:
        _atomic_torch_save(out, path)
    _barrier()


def load_consolidated(path: str, model, optimizer=None, features=None) -> int:
    """Cut this rank's shards out of a consolidated checkpoint (any grid)."""
    try:
        ck = torch.load(path, weights_only=False, map_location="cpu")
    except Exception as e:
        raise CheckpointError(f"cannot read {path}: {e}") from e
    with torch.no_grad():
        for l, layer in enumerate(model.layers):
            w = _cut_weight(layer, ck["weights"][l])
            layer.weight.copy_(w.to(layer.weight.device, layer.weight.dtype))
        if features is not None and ck.get("features") is not None:
            f = _cut_features(ck["features"], features)
            features.copy_(f.to(features.device, features.dtype))
    if optimizer is not None and ck.get("step", 0) > 0:
        def restore(p, avg, sq, master):
            st = optimizer._init_state(p)
            st["step"] = int(ck["step"])
            st["exp_avg"].copy_(avg.to(p.device))
            st["exp_avg_sq"].copy_(sq.to(p.device))
            if st.get("master") is not None and master is not None:
                st["master"].copy_(master.to(p.device))

        for l, layer in enumerate(model.layers):
            a, s = ck["moments"]["exp_avg"][l], ck["moments"]["exp_avg_sq"][l]
            if a is not None and s is not None:
                restore(layer.weight, _cut_weight(layer, a), _cut_weight(layer, s), None)
        if features is not None and ck.get("features_exp_avg") is not None:
            restore(
                features,
                _cut_features(ck["features_exp_avg"], features),
                _cut_features(ck["features_exp_avg_sq"], features),
                _cut_features(ck["features"], features),
            )
    return int(ck["epoch"]) + 1
