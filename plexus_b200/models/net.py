"""GCN models: the 3D-parallel ``Net`` and a serial single-process oracle.

``Net`` mirrors the example model of the reference (reference:
examples/train.py:55-79: ``num_gcn_layers`` GCNConv layers with ReLU between
them) with the layers registered in a ``ModuleList`` so that
``model.parameters()`` and ``state_dict()`` see the weights.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F

from ..ops.dropout import relu_dropout_2d
from .gcn_conv import GCNConv, GCNStackFunction, init_full_weight


class Net(torch.nn.Module):
    def __init__(self, num_gcn_layers, input_size, hidden_size, output_size, fuse_layers: bool = True,
                 seed: Optional[int] = None, order: str = "auto", dropout: float = 0.0):
        """``order``: per-layer multiplication order, see :class:`GCNConv` (``"auto"`` aggregates
        after the transform wherever that makes the sparse product narrower).
        ``dropout``: probability of dropping a hidden activation (after the ReLU, training mode only;
        the reference model has none).  The mask of an element depends on its position in the
        unsharded activation, the layer, the seed and the number of training steps taken, so every
        grid shape - and the serial model - drops the same elements."""
        super().__init__()
        self.num_gcn_layers = num_gcn_layers
        self.dropout = float(dropout)
        self.dropout_seed = 0 if seed is None else int(seed)
        self.steps_taken = 0
        self.fuse_layers = fuse_layers and self.dropout == 0.0
        dims = [input_size] + [hidden_size] * (num_gcn_layers - 1) + [output_size]
        self.dims = dims
        self.layers = torch.nn.ModuleList(
            GCNConv(dims[i], dims[i + 1], i, seed=seed, order=order if i > 0 else "aggregate_first")
            for i in range(num_gcn_layers)
        )

    def forward(self, x, edge_index_shards):
        L = self.num_gcn_layers
        if self.fuse_layers:
            specs, adjs = [], []
            for i, layer in enumerate(self.layers):
                pair = edge_index_shards[i % len(edge_index_shards)]
                specs.append(layer.spec(pair[0], relu=(i != L - 1)))
                adjs.append(pair)
            return GCNStackFunction.apply(specs, adjs, x, *[l.weight for l in self.layers])
        drop = self.dropout > 0 and self.training
        for i, layer in enumerate(self.layers):
            x = layer(x, edge_index_shards)
            if i != L - 1:
                if drop:
                    # the activation is sharded by rows over the layer's depth axis and by columns
                    # over its outer axis
                    x = relu_dropout_2d(x, self.dropout, dropout_seed(self.dropout_seed, i, self.steps_taken),
                                        layer.depth_rank * x.shape[0], layer.outer_rank * x.shape[1],
                                        layer.true_out_channels)
                else:
                    x = F.relu(x)
        if drop:
            self.steps_taken += 1
        return x


def dropout_seed(seed: int, layer: int, step: int) -> int:
    return (seed * 1000003 + layer * 7919 + step * 104729 + 17) % (1 << 62)


class SerialGCN(torch.nn.Module):
    """Single-process dense-weight GCN used as the numerical oracle.

    Uses the same weight initialisation as :class:`GCNConv`, so a parallel
    run with the same seed starts from the same parameters.
    """

    def __init__(self, num_gcn_layers, input_size, hidden_size, output_size, seed: Optional[int] = None,
                 dtype=torch.float32):
        super().__init__()
        dims = [input_size] + [hidden_size] * (num_gcn_layers - 1) + [output_size]
        self.weights = torch.nn.ParameterList(
            torch.nn.Parameter(init_full_weight(dims[i], dims[i + 1], i, seed).to(dtype))
            for i in range(num_gcn_layers)
        )

    @classmethod
    def from_consolidated(cls, path: str, dtype=torch.float32):
        """``(model, features)`` from a grid-independent checkpoint written by a parallel run
        (``utils.checkpoint.save_consolidated``): the trained weights, unpadded, and the trained
        input features in the processed (permuted) node order - for single-process evaluation or
        inference of a model that was trained on any grid."""
        ck = torch.load(path, weights_only=False, map_location="cpu")
        ws = [w.to(dtype) for w in ck["weights"]]
        model = cls.__new__(cls)
        torch.nn.Module.__init__(model)
        model.weights = torch.nn.ParameterList(torch.nn.Parameter(w.clone()) for w in ws)
        feats = ck.get("features")
        return model, (None if feats is None else feats.to(dtype))

    def forward(self, x, adjs: List[torch.Tensor], dropout: float = 0.0, seed: int = 0, step: int = 0):
        """``adjs[l % len(adjs)]`` is the (square, unsharded) adjacency used at layer ``l``.

        With ``dropout`` the same position-keyed masks as the parallel :class:`Net` (same ``seed``,
        ``step`` = number of training forwards taken) are applied."""
        L = len(self.weights)
        for l, w in enumerate(self.weights):
            A = adjs[l % len(adjs)]
            x = torch.sparse.mm(A, x) @ w
            if l != L - 1:
                if dropout > 0:
                    x = relu_dropout_2d(x, dropout, dropout_seed(seed, l, step), 0, 0, x.shape[1])
                else:
                    x = torch.relu(x)
        return x


def serial_loss(logits, labels, num_nodes):
    """Sum of cross-entropy over rows with a non-negative label, divided by ``num_nodes``."""
    return F.cross_entropy(logits, labels, ignore_index=-1, reduction="sum") / num_nodes
