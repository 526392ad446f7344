"""Per-rank loader: builds this rank's adjacency, feature and label shards.

Reference: plexus/utils/dataloader.py (``DataLoader(data_dir, num_gcn_layers)
.load()`` -> ``(adj_shards, features_flat, labels, num_nodes, num_features,
num_classes)``).  The sharding rules are the same:

* input features ``[N, F]``: rows over X, columns over Y (padded so the local
  width divides by Z), flattened row-major and 1-D sliced over Z;
* labels: rows over the depth axis of the last layer;
* adjacency for layer type ``t = layer % 3``: rows over the layer's depth
  axis, columns over its outer axis, i.e. (Z,X), (Y,Z), (X,Y); both ``A`` and
  ``A^T`` are returned as CSR.  With the double permutation, even layers use
  version 0 (``P A P2^T``) and odd layers version 1 (``P2 A P^T``).

Differences by design: shards are built with int32 indices, on the device
when one is present; identical shards are built once and shared; for a
symmetric graph the transposed shard is taken as the mirrored block of the
other version instead of being re-sorted; padded label rows are ``-1``
(ignored by the loss) instead of class 0; each version is paired with its own
edge weights; partition files are concatenated as int64.
"""

from __future__ import annotations

import glob
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from .. import runtime
from ..data import graph_ops
from ..data.container import Data, load_processed
from ..parallel.grid import axis_roles, default_device, get_grid, loss_axes
from ..parallel.sharding import block_range, pad_dimension, padded_channels


class DataLoader:
    def __init__(
        self,
        data_dir: Optional[str],
        num_gcn_layers: int,
        *,
        data: Optional[Tuple[object, int]] = None,
        source=None,
        device: Optional[torch.device] = None,
        dtype: Optional[torch.dtype] = None,
        keep_masks: bool = True,
    ):
        """
        Args:
            data_dir: directory with one processed ``.pt`` file or a partition tree
            num_gcn_layers: number of GCN layers in the model
            data: optional in-memory ``(data, num_classes)`` instead of files
            source: optional generator object (``data.sharded_synthetic.ShardedSyntheticGraph``)
                that produces this rank's blocks directly; no global edge list exists then
        """
        self.data_dir = data_dir
        self.num_gcn_layers = num_gcn_layers
        self._in_memory = data
        self.source = source
        self.device = device if device is not None else default_device()
        self.dtype = dtype if dtype is not None else runtime.flags.dtype
        self.keep_masks = keep_masks
        self.masks: Dict[str, torch.Tensor] = {}
        self.symmetric = False
        self.partitioned = False
        self.double_perm = False
        if source is not None:
            self.double_perm = bool(source.double_perm)
        elif data is None:
            self.partitioned = os.path.exists(os.path.join(data_dir, "metadata.pt"))
            self.double_perm = os.path.exists(os.path.join(data_dir, "edge_index", "1"))
            self.labels_dir = os.path.join(data_dir, "output_labels")
            self.num_partitions_dim = len(glob.glob(os.path.join(self.labels_dir, "0", "*.pt")))
            self.adj_dir = os.path.join(data_dir, "edge_index")
            self.features_dir = os.path.join(data_dir, "input_features")
        else:
            self.double_perm = hasattr(data[0], "edge_index_2")

    # ------------------------------------------------------------------ plan
    def _plan(self) -> None:
        g = get_grid()
        N, Fdim = self.num_nodes, self.num_features
        align = runtime.flags.channel_align
        # features: rows over X, columns over Y, flat slice over Z
        self.nodes_start, self.nodes_stop = block_range(N, g.X, g.coord("x"))
        f_pad = padded_channels(Fdim, g.Y, g.Z, align)
        f_step = f_pad // g.Y
        self.features_start, self.features_stop = g.coord("y") * f_step, (g.coord("y") + 1) * f_step
        local_elems = (self.nodes_stop - self.nodes_start) * f_step
        d_step = pad_dimension(local_elems, g.Z) // g.Z
        self.depth_start, self.depth_stop = g.coord("z") * d_step, (g.coord("z") + 1) * d_step
        # labels: rows over the row axis of the logits
        row_axis, _ = loss_axes(self.num_gcn_layers)
        self.labels_start, self.labels_stop = block_range(N, g.size(row_axis), g.coord(row_axis))
        # adjacency ranges per layer type
        self.adj_ranges = []
        for t in range(3):
            outer, _inner, depth = axis_roles(t)
            r0, r1 = block_range(N, g.size(depth), g.coord(depth))
            c0, c1 = block_range(N, g.size(outer), g.coord(outer))
            self.adj_ranges.append((r0, r1, c0, c1))

    # ------------------------------------------------------- partition files
    def _part_span(self, start: int, stop: int, size: int) -> range:
        p = self.num_partitions_dim
        return range(min(start // size, p), min((stop - 1) // size + 1, p))

    def _load_adj_blocks(self, version: int, r0: int, r1: int, c0: int, c1: int):
        size = pad_dimension(self.num_nodes, self.num_partitions_dim) // self.num_partitions_dim
        eis, ews = [], []
        for i in self._part_span(r0, r1, size):
            for j in self._part_span(c0, c1, size):
                path = os.path.join(self.adj_dir, str(version), f"{i}_{j}.pt")
                if not os.path.exists(path):
                    raise FileNotFoundError(f"missing partition file {path}")
                try:
                    ei, ew = torch.load(path, weights_only=False)
                except Exception as e:
                    raise RuntimeError(f"corrupt partition file {path}: {e}") from e
                eis.append(ei.to(torch.int64))
                ews.append(ew.to(torch.float32))
        if not eis:
            return torch.empty((2, 0), dtype=torch.int64), torch.empty(0, dtype=torch.float32)
        return torch.cat(eis, dim=1), torch.cat(ews, dim=0)

    def _load_feature_blocks(self):
        p = self.num_partitions_dim
        size_n = pad_dimension(self.num_nodes, p) // p
        size_f = pad_dimension(self.num_features, p) // p
        rows = []
        span_i = self._part_span(self.nodes_start, self.nodes_stop, size_n)
        span_j = self._part_span(self.features_start, self.features_stop, size_f)
        for i in span_i:
            cols = [torch.load(os.path.join(self.features_dir, f"{i}_{j}.pt"), weights_only=False) for j in span_j]
            if cols:
                rows.append(torch.cat(cols, dim=1))
        origin = (
            (span_i.start * size_n) if len(span_i) else self.nodes_start,
            (span_j.start * size_f) if len(span_j) else self.features_start,
        )
        if not rows or rows[0].numel() == 0 and len(rows) == 1:
            return torch.zeros((0, 0)), origin
        return torch.cat(rows, dim=0), origin

    def _load_label_blocks(self, version: int):
        p = self.num_partitions_dim
        size = pad_dimension(self.num_nodes, p) // p
        span = self._part_span(self.labels_start, self.labels_stop, size)
        parts = [torch.load(os.path.join(self.labels_dir, str(version), f"{i}.pt"), weights_only=False) for i in span]
        origin = span.start * size if len(span) else self.labels_start
        if not parts:
            return torch.empty(0, dtype=torch.int64), origin
        return torch.cat([q.to(torch.int64) for q in parts]), origin

    # ----------------------------------------------------------- shard build
    def _edges_of(self, version: int, r0, r1, c0, c1):
        """(edge_index, edge_weight, sorted_by_row) covering the requested block."""
        if self.partitioned:
            ei, ew = self._load_adj_blocks(version, r0, r1, c0, c1)
            return ei.to(self.device), ew.to(self.device), False
        if version not in self._edge_cache:
            d = self.data
            ei = d.edge_index if version == 0 else d.edge_index_2
            ew = d.edge_weight if version == 0 else d.edge_weight_2
            ei = ei.to(self.device)
            ew = ew.to(self.device, torch.float32)
            srt = bool((ei[0, 1:] >= ei[0, :-1]).all()) if ei.shape[1] > 1 else True
            self._edge_cache = {version: (ei, ew, srt)}  # keep one version resident
        return self._edge_cache[version]

    def _csr_block(self, version: int, r0, r1, c0, c1) -> torch.Tensor:
        key = (version, r0, r1, c0, c1)
        if key not in self._csr_cache:
            ei, ew, srt = self._edges_of(version, r0, r1, c0, c1)
            row, col, val = graph_ops.extract_block(ei, ew, r0, r1, c0, c1, sorted_by_row=srt)
            crow, col, val = graph_ops.coo_to_csr(row, col, val, r1 - r0, c1 - c0)
            self._csr_cache[key] = graph_ops.csr_tensor(crow, col, val, (r1 - r0, c1 - c0))
        return self._csr_cache[key]

    def _adj_pair(self, shard_idx: int):
        version = shard_idx % 2 if self.double_perm else 0
        r0, r1, c0, c1 = self.adj_ranges[shard_idx % 3]
        A = self._csr_block(version, r0, r1, c0, c1)
        if self.symmetric:
            # (P A P2^T)^T = P2 A P^T for symmetric A: the transposed shard is
            # the mirrored block of the other version.
            tv = (1 - version) if self.double_perm else version
            At = self._csr_block(tv, c0, c1, r0, r1)
        else:
            tkey = ("T", version, r0, r1, c0, c1)
            if tkey not in self._csr_cache:
                self._csr_cache[tkey] = graph_ops.csr_transpose(A)
            At = self._csr_cache[tkey]
        return A, At

    def _feature_shard(self, x: torch.Tensor, origin=(0, 0)) -> torch.Tensor:
        rows = self.nodes_stop - self.nodes_start
        cols = self.features_stop - self.features_start
        r0, c0 = self.nodes_start - origin[0], self.features_start - origin[1]
        if x.numel() == 0:
            local = torch.zeros((rows, cols), dtype=torch.float32)
        else:
            local = x[max(r0, 0) : max(r0 + rows, 0), max(c0, 0) : max(c0 + cols, 0)]
            local = F.pad(local, (0, cols - local.shape[1], 0, rows - local.shape[0]))
        flat = local.reshape(-1)
        need = self.depth_stop - flat.numel()
        if need > 0:
            flat = F.pad(flat, (0, need))
        flat = flat[self.depth_start : self.depth_stop]
        return flat.to(self.device, self.dtype).contiguous().requires_grad_()

    def _label_shard(self, y: torch.Tensor, origin: int = 0) -> torch.Tensor:
        n = self.labels_stop - self.labels_start
        s = self.labels_start - origin
        local = y[max(s, 0) : max(s + n, 0)].to(torch.int64)
        local = F.pad(local, (0, n - local.shape[0]), value=-1)
        return local.to(self.device)

    # ------------------------------------------------------------------ load
    def load(self):
        """Return ``(adj_shards, features, labels, num_nodes, num_features, num_classes)``."""
        self._edge_cache: Dict[int, tuple] = {}
        self._csr_cache: Dict[tuple, torch.Tensor] = {}
        with torch.no_grad():
            if self.source is not None:
                src = self.source
                self.num_nodes, self.num_features, self.num_classes = src.num_nodes, src.num_features, src.num_classes
                self.symmetric, self.double_perm = bool(src.symmetric), bool(src.double_perm)
                self.data = None
            elif self.partitioned:
                self.num_nodes, self.num_features, self.num_classes = torch.load(
                    os.path.join(self.data_dir, "metadata.pt"), weights_only=False
                )
                extra = os.path.join(self.data_dir, "extra.pt")
                if os.path.exists(extra):
                    self.symmetric = bool(torch.load(extra, weights_only=False).get("symmetric", False))
                self.data = None
            else:
                if self._in_memory is not None:
                    self.data, self.num_classes = self._in_memory
                else:
                    pt = [f for f in os.listdir(self.data_dir) if f.endswith(".pt")]
                    if len(pt) != 1:
                        raise ValueError("Expected exactly one .pt file in the directory.")
                    self.data, self.num_classes = load_processed(os.path.join(self.data_dir, pt[0]))
                self.num_nodes, self.num_features = int(self.data.x.shape[0]), int(self.data.x.shape[1])
                self.symmetric = bool(getattr(self.data, "symmetric", False))
                # a single processed file says by its contents whether it carries both versions
                self.double_perm = hasattr(self.data, "edge_index_2")
            self._plan()

            n_shards = min(6 if self.double_perm else 3, self.num_gcn_layers)
            # build version 0 blocks first, then version 1, so only one global
            # edge list is resident on the device at a time
            order = sorted(range(n_shards), key=lambda i: (i % 2 if self.double_perm else 0, i))
            pairs = {}
            if self.source is not None:
                # every block this rank needs, generated in one pass over the raw edge stream
                need = []
                for i in range(n_shards):
                    v = i % 2 if self.double_perm else 0
                    r0, r1, c0, c1 = self.adj_ranges[i % 3]
                    need.append((v, r0, r1, c0, c1))
                    need.append(((1 - v) if self.double_perm else v, c0, c1, r0, r1))  # its transpose
                self._csr_cache.update(self.source.build_blocks(need))
            elif self.symmetric and self.double_perm:
                # both members of a pair come from different versions; warm the
                # cache version by version
                for v in (0, 1):
                    for i in range(n_shards):
                        r0, r1, c0, c1 = self.adj_ranges[i % 3]
                        if i % 2 == v:
                            self._csr_block(v, r0, r1, c0, c1)
                        else:
                            self._csr_block(v, c0, c1, r0, r1)
            for i in order:
                pairs[i] = self._adj_pair(i)
            adj_shards = [pairs[i] for i in range(n_shards)]
            self._edge_cache = {}

            use_second = self.double_perm and self.num_gcn_layers % 2 == 0
            if self.source is not None:
                src = self.source
                x = src.feature_block(self.nodes_start, self.nodes_stop, self.features_start, self.features_stop)
                features = self._feature_shard(x, (self.nodes_start, self.features_start))
                del x
                ver = 1 if use_second else 0
                labels = self._label_shard(src.labels(ver, self.labels_start, self.labels_stop), self.labels_start)
                if self.keep_masks:
                    n = self.labels_stop - self.labels_start
                    for m in ("train_mask", "val_mask", "test_mask"):
                        loc = src.mask(m, ver, self.labels_start, self.labels_stop)
                        self.masks[m] = F.pad(loc, (0, n - loc.shape[0]), value=False).to(self.device)
            elif self.partitioned:
                x, origin = self._load_feature_blocks()
                features = self._feature_shard(x, origin)
                y, yo = self._load_label_blocks(1 if use_second else 0)
                labels = self._label_shard(y, yo)
            else:
                features = self._feature_shard(self.data.x)
                labels = self._label_shard(self.data.y_2 if use_second else self.data.y)
                if self.keep_masks:
                    for m in ("train_mask", "val_mask", "test_mask"):
                        name = m + "_2" if use_second else m
                        if hasattr(self.data, name):
                            mk = getattr(self.data, name)
                            n = self.labels_stop - self.labels_start
                            loc = mk[self.labels_start : self.labels_stop].to(torch.bool)
                            self.masks[m] = F.pad(loc, (0, n - loc.shape[0]), value=False).to(self.device)
            self._csr_cache = {}
            return (
                adj_shards,
                features,
                labels,
                self.num_nodes,
                self.num_features,
                self.num_classes,
            )
