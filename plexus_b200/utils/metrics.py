"""JSON-lines metrics sink: one record per epoch / event, written by rank 0.

Records carry what the stdout log of the reference cannot: device-timed epoch
milliseconds (max over ranks), per-region times, bytes handed to each
collective, nnz balance of the adjacency shards and peak device memory.
"""

from __future__ import annotations

import json
import os
import time
from typing import Optional

import torch
import torch.distributed as dist


class MetricsSink:
    def __init__(self, path: Optional[str]):
        self.path = path
        self._is_root = not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
        if path and self._is_root:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            self._f = open(path, "a")
        else:
            self._f = None

    def log(self, **record) -> None:
        if self._f is None:
            return
        record.setdefault("ts", time.time())
        self._f.write(json.dumps(record) + "\n")
        self._f.flush()

    def close(self) -> None:
        if self._f is not None:
            self._f.close()
            self._f = None


def max_over_ranks(value: float) -> float:
    """Maximum of a host scalar over all ranks (identity without a process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def shard_nnz_imbalance(adj_shards) -> float:
    """max/mean of the nnz of this rank's first adjacency shard over all ranks."""
    nnz = float(adj_shards[0][0].values().numel())
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return 1.0
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([nnz, nnz], dtype=torch.float64, device=dev)
    mx, sm = t[:1].clone(), t[1:].clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    mean = sm.item() / dist.get_world_size()
    return mx.item() / mean if mean > 0 else 1.0


def peak_memory_gb() -> float:
    if torch.cuda.is_available():
        return torch.cuda.max_memory_allocated() / 1024**3
    return 0.0
