"""Minimal graph container with the attribute names of a PyG ``Data`` object.

Processed-graph files are ``torch.save((data, num_classes))`` where ``data``
carries ``x [N,F]``, ``y [N]`` (int64, -1 = unlabeled), ``edge_index [2,E]``
(int64), ``edge_weight [E]`` and, with the double permutation,
``edge_index_2``, ``edge_weight_2`` and ``y_2`` (reference:
plexus/utils/dataset.py:205-246).  PyTorch Geometric is optional: this class
stands in for its ``Data`` when it is not installed, and anything exposing the
same attributes (a real PyG object included) is accepted by the loaders.
"""

from __future__ import annotations

from typing import Any, Dict, Iterator

import torch


class Data:
    def __init__(self, **kwargs: Any):
        for k, v in kwargs.items():
            setattr(self, k, v)

    # -- dict-like helpers -------------------------------------------------
    def keys(self):
        return [k for k in self.__dict__ if not k.startswith("_")]

    def __contains__(self, key: str) -> bool:
        return key in self.__dict__

    def __iter__(self) -> Iterator:
        for k in self.keys():
            yield k, getattr(self, k)

    def to_dict(self) -> Dict[str, Any]:
        return {k: getattr(self, k) for k in self.keys()}

    @property
    def num_nodes(self) -> int:
        if "_num_nodes" in self.__dict__ and self.__dict__["_num_nodes"] is not None:
            return int(self.__dict__["_num_nodes"])
        x = self.__dict__.get("x")
        if x is not None:
            return int(x.shape[0])
        ei = self.__dict__.get("edge_index")
        if ei is not None and ei.numel():
            return int(ei.max().item()) + 1
        return 0

    @num_nodes.setter
    def num_nodes(self, n) -> None:
        self.__dict__["_num_nodes"] = n

    @property
    def num_edges(self) -> int:
        ei = self.__dict__.get("edge_index")
        return 0 if ei is None else int(ei.shape[1])

    def to(self, device) -> "Data":
        out = Data()
        for k, v in self.__dict__.items():
            out.__dict__[k] = v.to(device) if torch.is_tensor(v) else v
        return out

    def __repr__(self) -> str:
        parts = []
        for k in self.keys():
            v = getattr(self, k)
            parts.append(f"{k}={list(v.shape)}" if torch.is_tensor(v) else f"{k}={v!r}")
        return "Data(" + ", ".join(parts) + ")"


def load_processed(path: str):
    """Load ``(data, num_classes)`` written by :func:`save_processed` or by the reference."""
    obj = torch.load(path, weights_only=False)
    if isinstance(obj, tuple) and len(obj) == 2:
        return obj
    return obj, None


def save_processed(data, num_classes: int, path: str) -> None:
    import os

    tmp = path + ".tmp"
    torch.save((data, num_classes), tmp)
    os.replace(tmp, path)
