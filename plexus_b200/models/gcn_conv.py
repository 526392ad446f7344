"""3D tensor-parallel GCN convolution: ``OUT = (A . H) . W`` on an X x Y x Z grid.

Per layer the grid axes play the roles (outer, inner, depth), rotating with
the layer index.  Every rank holds

* ``A``  : rows by depth rank, columns by outer rank (and ``A^T`` for backward),
* ``H``  : rows by outer rank, columns by inner rank (layer 0: additionally
  flattened and sliced over depth, gathered before use),
* ``W``  : rows by inner rank, columns by outer rank, flattened and sliced over
  depth when divisible,

so ``AGG = A.H`` is a partial sum over the outer axis and ``OUT = AGG.W`` a
partial sum over the inner axis; ``OUT`` is laid out exactly like the next
layer's ``H``.

Forward and backward follow the reference's autograd function (reference:
plexus/gcn_conv.py:131-296, module :299-411, blocked aggregation :67-128).
Two structural additions:

* an optional fused ReLU: the activation is applied where the layer output is
  produced (GEMM epilogue, or right after the inner-axis reduction), and its
  derivative mask is applied where the gradient is produced (the epilogue of
  the previous layer's backward SpMM), so no separate elementwise pass runs;
* :class:`GCNStackFunction` runs all layers inside one autograd node so those
  fusions can cross layer boundaries.

With ``runtime.flags.comm == "fused"`` the aggregation/combination collectives
are carried out by kernels that access peer memory (``parallel.fused``)
instead of NCCL calls.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch.nn import Parameter

from .. import ops, runtime
from ..parallel import collectives as coll
from ..parallel.grid import get_grid, group_rank, group_size
from ..parallel.sharding import (
    depth_slice,
    extract_local_params_from_full_params,
    pad_dimension,
    padded_channels,
    shard_2d,
)
from ..utils.matmul_tuning import tuned_matmul
from ..utils.timers import get_timers

MAX_ROWS_PER_CHUNK = 1_000_000


def extract_csr_submatrix(csr_matrix, start_row, end_row):
    """Row chunk ``[start_row, end_row)`` of a CSR matrix."""
    return ops.extract_csr_submatrix(csr_matrix, start_row, end_row)


def chunked_spmm_all_reduce(csr_matrix, H, ar_group, max_rows_per_chunk: Optional[int] = None):
    """Row-blocked ``A.H`` with one all-reduce per block.

    With ``overlap_agg`` the all-reduce of block k runs asynchronously while
    block k+1 is multiplied.  Blocks are row *ranges* of the same CSR arrays,
    so no sub-matrix is materialised and nothing synchronises with the host.
    """
    timers = get_timers()
    overlap = runtime.flags.overlap_agg
    if overlap:
        timers.start("AGG = A * H and All-Reduce AGG")
    num_rows = csr_matrix.shape[0]
    cap = max_rows_per_chunk or MAX_ROWS_PER_CHUNK
    num_chunks = max(1, (num_rows + cap - 1) // cap)
    rows_per_chunk = num_rows // num_chunks
    AGG = torch.empty((num_rows, H.shape[1]), dtype=H.dtype, device=H.device)
    handles = []
    p = group_size(ar_group)
    for i in range(num_chunks):
        r0 = i * rows_per_chunk
        r1 = num_rows if i == num_chunks - 1 else (i + 1) * rows_per_chunk
        if not overlap:
            timers.start("AGG = A * H")
        ops.spmm(csr_matrix, H, row_range=(r0, r1), out=AGG[r0:r1])
        if not overlap:
            timers.stop("AGG = A * H")
        if p > 1 and not runtime.flags.skip_collectives:
            if overlap:
                handles.append(dist.all_reduce(AGG[r0:r1], group=ar_group, async_op=True))
            else:
                coll.all_reduce(AGG[r0:r1], ar_group)
    for h in handles:
        h.wait()
    if overlap:
        timers.stop("AGG = A * H and All-Reduce AGG")
    return AGG


@dataclass
class LayerSpec:
    """Static description of one layer on this rank."""

    layer_num: int
    local_features_shape: Tuple[int, int]
    local_weight_shape: Tuple[int, int]
    depth_group: object
    outer_group: object
    inner_group: object
    gather_features: bool
    gather_weights: bool
    relu: bool = False
    # transform-then-aggregate order: OUT = A . (H . W) with W holding all output columns
    combine_first: bool = False
    local_out_channels: int = 0


def _aggregate(A, H, spec: LayerSpec):
    timers = get_timers()
    if runtime.flags.comm == "fused" and group_size(spec.outer_group) > 1:
        from ..parallel import fused

        timers.start("AGG = A * H and All-Reduce AGG")
        AGG = fused.spmm_all_reduce(A, H, spec.outer_group)
        timers.stop("AGG = A * H and All-Reduce AGG")
        return AGG
    if runtime.flags.block_agg:
        return chunked_spmm_all_reduce(A, H, spec.outer_group)
    timers.start("AGG = A * H")
    AGG = ops.spmm(A, H)
    timers.stop("AGG = A * H")
    coll.all_reduce(AGG, spec.outer_group)
    return AGG


def _full_weight(weight, spec: LayerSpec, dtype):
    W = coll.all_gather(weight, dim=0, process_group=spec.depth_group) if spec.gather_weights else weight
    W = W.reshape(spec.local_weight_shape)
    return W if W.dtype == dtype else W.to(dtype)


def _combine_first_forward(H, A, weight, spec: LayerSpec):
    """``OUT = A . (H . W)``: cheaper when the layer narrows (few output channels).

    ``W`` is sharded by rows over the inner axis only, so ``T = H . W`` (partial over inner)
    has all output columns; ``A . T`` is partial over the outer axis and is reduce-scattered
    along the columns, which lands exactly in the standard output layout
    ``(N/depth) x (out/outer)``.  Returns ``(OUT, H)`` (the input is what backward needs).
    """
    timers = get_timers()
    timers.start("gcn conv fwd")
    W = _full_weight(weight, spec, H.dtype)
    timers.start("OUT = AGG * W")
    if runtime.flags.comm == "fused" and group_size(spec.inner_group) > 1:
        from ..parallel import fused

        T = fused.gemm_all_reduce(H, W, spec.inner_group)  # push fused in the GEMM epilogue
        timers.stop("OUT = AGG * W")
    else:
        T = tuned_matmul(H, W, "H * W " + str(spec.layer_num))
        timers.stop("OUT = AGG * W")
        coll.all_reduce(T, spec.inner_group)
    outer_p = group_size(spec.outer_group)
    if runtime.flags.comm == "fused" and outer_p > 1:
        from ..parallel import fused

        timers.start("AGG = A * H and All-Reduce AGG")
        U = fused.spmm_all_reduce(A, T, spec.outer_group)
        timers.stop("AGG = A * H and All-Reduce AGG")
    else:
        timers.start("AGG = A * H")
        U = ops.spmm(A, T)
        timers.stop("AGG = A * H")
        coll.all_reduce(U, spec.outer_group)
    lo = spec.local_out_channels
    r = group_rank(spec.outer_group)
    OUT = U if outer_p == 1 else U[:, r * lo : (r + 1) * lo].contiguous()
    if spec.relu:
        OUT = torch.relu_(OUT)
    timers.stop("gcn conv fwd")
    return OUT, H


def _combine_first_backward(grad_out, H, weight, A_t, spec: LayerSpec, input_relu_mask=None,
                            need_input_grad: bool = True):
    timers = get_timers()
    timers.start("gcn conv bwd")
    W = _full_weight(weight, spec, H.dtype)
    outer_p = group_size(spec.outer_group)
    depth_p = group_size(spec.depth_group)
    if outer_p > 1:
        # column blocks of the output gradient from every outer rank
        parts = coll.all_gather(grad_out.unsqueeze(0).contiguous(), dim=0, process_group=spec.outer_group)
        grad_u = parts.permute(1, 0, 2).reshape(grad_out.shape[0], -1).contiguous()
    else:
        grad_u = grad_out
    timers.start("GRAD_H = A.T * GRAD_AGG")
    if runtime.flags.comm == "fused" and depth_p > 1:
        from ..parallel import fused

        grad_t = fused.spmm_all_reduce(A_t, grad_u, spec.depth_group)
        timers.stop("GRAD_H = A.T * GRAD_AGG")
    else:
        grad_t = ops.spmm(A_t, grad_u)
        timers.stop("GRAD_H = A.T * GRAD_AGG")
        coll.all_reduce(grad_t, spec.depth_group)

    timers.start("GRAD_W = AGG.T * GRAD_OUT")
    grad_w = tuned_matmul(
        H, grad_t, "H.T * GRAD_T " + str(spec.layer_num), trans_a=True,
        out_dtype=torch.promote_types(weight.dtype, torch.float32),
    )
    timers.stop("GRAD_W = AGG.T * GRAD_OUT")
    coll.all_reduce(grad_w, spec.outer_group)  # rows of H are spread over the outer axis
    grad_w = grad_w.reshape(-1)
    if spec.gather_weights:
        # identical on every depth rank already: keep this rank's flat slice
        grad_w = depth_slice(grad_w, depth_p, group_rank(spec.depth_group)).clone()
    grad_w = grad_w.to(weight.dtype)

    grad_x = None
    if need_input_grad:
        timers.start("GRAD_AGG = GRAD_OUT * W.T")
        # the ReLU derivative of the layer input is applied in the GEMM epilogue
        grad_x = tuned_matmul(grad_t, W, "GRAD_T * W.T " + str(spec.layer_num), trans_b=True,
                              relu_mask=input_relu_mask)
        timers.stop("GRAD_AGG = GRAD_OUT * W.T")
    timers.stop("gcn conv bwd")
    return grad_x, grad_w


def layer_forward(x, A, weight, spec: LayerSpec):
    """Returns ``(OUT, saved)``; ``OUT`` already has the ReLU applied if ``spec.relu``.

    ``saved`` is what backward needs besides the weight: ``AGG`` for the aggregate-first order,
    the layer input for the combine-first order.
    """
    if spec.combine_first:
        return _combine_first_forward(x, A, weight, spec)
    timers = get_timers()
    timers.start("gcn conv fwd")
    if spec.gather_features:
        H = coll.all_gather(x, dim=0, process_group=spec.depth_group)
        n = spec.local_features_shape[0] * spec.local_features_shape[1]
        H = H[:n].reshape(spec.local_features_shape)
    else:
        H = x
    AGG = _aggregate(A, H, spec)
    W = _full_weight(weight, spec, AGG.dtype)

    inner_p = group_size(spec.inner_group)
    if runtime.flags.comm == "fused" and inner_p > 1:
        from ..parallel import fused

        timers.start("OUT = AGG * W")
        OUT = fused.gemm_all_reduce(AGG, W, spec.inner_group, relu=spec.relu)
        timers.stop("OUT = AGG * W")
    else:
        fuse_relu = spec.relu and inner_p == 1
        timers.start("OUT = AGG * W")
        OUT = tuned_matmul(AGG, W, "AGG * W " + str(spec.layer_num), relu=fuse_relu)
        timers.stop("OUT = AGG * W")
        coll.all_reduce(OUT, spec.inner_group)
        if spec.relu and not fuse_relu:
            OUT = torch.relu_(OUT)
    timers.stop("gcn conv fwd")
    return OUT, AGG


def layer_backward(grad_out, AGG, weight, A_t, spec: LayerSpec, input_relu_mask=None,
                   need_input_grad: bool = True):
    """Backward of one layer.

    ``grad_out`` must already carry this layer's own ReLU derivative.
    ``input_relu_mask`` (the layer's input when that input is a ReLU output)
    is applied to the returned input gradient inside the SpMM epilogue.
    Returns ``(grad_x, grad_weight_flat)``.
    """
    if spec.combine_first:
        return _combine_first_backward(grad_out, AGG, weight, A_t, spec, input_relu_mask, need_input_grad)
    timers = get_timers()
    timers.start("gcn conv bwd")
    W = _full_weight(weight, spec, AGG.dtype)

    timers.start("GRAD_W = AGG.T * GRAD_OUT")
    grad_w = tuned_matmul(
        AGG, grad_out, "AGG.T * GRAD_OUT " + str(spec.layer_num), trans_a=True,
        out_dtype=torch.promote_types(weight.dtype, torch.float32),
    )
    timers.stop("GRAD_W = AGG.T * GRAD_OUT")
    # the reduction over the depth axis overlaps the rest of this layer's backward
    pending_w = coll.reduce_grad_async(grad_w.reshape(-1), spec.depth_group, scatter=spec.gather_weights)

    if not need_input_grad:
        grad_w = pending_w.wait().reshape(-1).to(weight.dtype)
        timers.stop("gcn conv bwd")
        return None, grad_w

    outer_p = group_size(spec.outer_group)
    timers.start("GRAD_AGG = GRAD_OUT * W.T")
    if runtime.flags.comm == "fused" and outer_p > 1:
        from ..parallel import fused

        grad_agg = fused.gemm_all_reduce(grad_out, W, spec.outer_group, trans_b=True)
        timers.stop("GRAD_AGG = GRAD_OUT * W.T")
    else:
        grad_agg = tuned_matmul(grad_out, W, "GRAD_OUT * W.T " + str(spec.layer_num), trans_b=True)
        timers.stop("GRAD_AGG = GRAD_OUT * W.T")
        coll.all_reduce(grad_agg, spec.outer_group)

    depth_p = group_size(spec.depth_group)
    timers.start("GRAD_H = A.T * GRAD_AGG")
    if runtime.flags.comm == "fused" and depth_p > 1:
        from ..parallel import fused

        grad_x = None
        if spec.gather_features:
            # the features are a flat depth shard: only this rank's row segment of the reduced
            # gradient is needed, so the epilogue reduce-scatters instead of all-reducing
            seg = fused.spmm_reduce_scatter(A_t, grad_agg, spec.depth_group, relu_mask=input_relu_mask)
            if seg is not None:
                grad_x = seg.reshape(-1).clone()
        if grad_x is None:
            grad_x = fused.spmm_all_reduce(A_t, grad_agg, spec.depth_group, relu_mask=input_relu_mask)
            if spec.gather_features:
                flat = grad_x.reshape(-1)
                pad = (-flat.numel()) % depth_p
                if pad:
                    flat = torch.nn.functional.pad(flat, (0, pad))
                grad_x = depth_slice(flat, depth_p, group_rank(spec.depth_group)).clone()
        timers.stop("GRAD_H = A.T * GRAD_AGG")
    else:
        grad_x = ops.spmm(A_t, grad_agg, relu_mask=input_relu_mask)
        timers.stop("GRAD_H = A.T * GRAD_AGG")
        if spec.gather_features:
            flat = grad_x.reshape(-1)
            pad = (-flat.numel()) % depth_p
            if pad:
                flat = torch.nn.functional.pad(flat, (0, pad))
            grad_x = coll.reduce_scatter(flat, dim=0, process_group=spec.depth_group)
        else:
            coll.all_reduce(grad_x, spec.depth_group)
    grad_w = pending_w.wait().reshape(-1).to(weight.dtype)
    timers.stop("gcn conv bwd")
    return grad_x, grad_w


class GCNConvFunction(torch.autograd.Function):
    """One 3D-parallel GCN layer as an autograd node."""

    @staticmethod
    def forward(
        ctx,
        x,
        edge_index,
        edge_index_t,
        weight,
        local_features_shape,
        local_weight_shape,
        all_gather_group,
        aggregation_all_reduce_group,
        combination_all_reduce_group,
        gather_features,
        gather_weights,
        layer_num,
        relu=False,
        combine_first=False,
        local_out_channels=0,
    ):
        spec = LayerSpec(
            layer_num=layer_num,
            local_features_shape=tuple(local_features_shape),
            local_weight_shape=tuple(local_weight_shape),
            depth_group=all_gather_group,
            outer_group=aggregation_all_reduce_group,
            inner_group=combination_all_reduce_group,
            gather_features=bool(gather_features),
            gather_weights=bool(gather_weights),
            relu=bool(relu),
            combine_first=bool(combine_first),
            local_out_channels=int(local_out_channels),
        )
        OUT, AGG = layer_forward(x, edge_index, weight, spec)
        ctx.spec = spec
        ctx.adj_t = edge_index_t
        if spec.relu:
            ctx.save_for_backward(AGG, weight, OUT)
        else:
            ctx.save_for_backward(AGG, weight)
        ctx.need_x = x.requires_grad
        return OUT

    @staticmethod
    def backward(ctx, grad_output):
        spec = ctx.spec
        if spec.relu:
            AGG, weight, OUT = ctx.saved_tensors
            grad_output = ops.relu_backward(grad_output.contiguous(), OUT)
        else:
            AGG, weight = ctx.saved_tensors
            grad_output = grad_output.contiguous()
        grad_x, grad_w = layer_backward(
            grad_output, AGG, weight, ctx.adj_t, spec, need_input_grad=ctx.need_x
        )
        return (grad_x, None, None, grad_w) + (None,) * 11


class GCNStackFunction(torch.autograd.Function):
    """All layers of a GCN in one autograd node (ReLU between layers fused).

    ``args`` = (features, w_0, ..., w_{L-1}); ``specs`` / ``adjs`` are the
    per-layer :class:`LayerSpec` and ``(A, A^T)`` pairs.
    """

    @staticmethod
    def forward(ctx, specs: Sequence[LayerSpec], adjs, x, *weights):
        saved = []
        h = x
        for spec, (A, _A_t), w in zip(specs, adjs, weights):
            out, agg = layer_forward(h, A, w, spec)
            saved.append((agg, out))
            h = out
        ctx.specs, ctx.adjs = specs, adjs
        ctx.num_layers = len(specs)
        flat = []
        for agg, out in saved:
            flat += [agg, out]
        ctx.save_for_backward(*flat, *weights)
        ctx.need_x = x.requires_grad
        return h

    @staticmethod
    def backward(ctx, grad_output):
        L = ctx.num_layers
        tensors = ctx.saved_tensors
        aggs = tensors[0 : 2 * L : 2]
        outs = tensors[1 : 2 * L : 2]
        weights = tensors[2 * L :]
        grad_ws: List[Optional[torch.Tensor]] = [None] * L
        g = grad_output.contiguous()
        last = ctx.specs[L - 1]
        if last.relu:
            g = ops.relu_backward(g, outs[L - 1])
        grad_x = None
        for l in range(L - 1, -1, -1):
            spec = ctx.specs[l]
            # the input of layer l is the ReLU output of layer l-1
            mask = outs[l - 1] if (l > 0 and ctx.specs[l - 1].relu) else None
            need = l > 0 or ctx.need_x
            g, grad_ws[l] = layer_backward(
                g, aggs[l], weights[l], ctx.adjs[l][1], spec, input_relu_mask=mask, need_input_grad=need
            )
        grad_x = g
        return (None, None, grad_x, *grad_ws)


WEIGHT_STREAM = 500  # hash stream of layer l is WEIGHT_STREAM + l


def _weight_seed(seed: Optional[int]) -> int:
    return (torch.initial_seed() if seed is None else seed) % (1 << 62)


def init_full_weight(in_channels: int, out_channels: int, layer_num: int, seed: Optional[int] = None):
    """Kaiming-uniform (a=sqrt(5)) ``[in, out]`` matrix, identical on every rank and grid.

    ``fan_in`` is the number of input channels, so the bound is ``1/sqrt(in_channels)``.  Entry
    ``(r, c)`` is a counter-based hash of ``(seed, layer, r * out + c)``: the values do not depend
    on the grid shape, and a rank can produce just its shard (:func:`init_weight_shard`).
    """
    from ..data.synthetic import uniform01

    bound = 1.0 / math.sqrt(in_channels) if in_channels > 0 else 0.0
    idx = torch.arange(in_channels * out_channels, dtype=torch.int64)
    u = uniform01(_weight_seed(seed), WEIGHT_STREAM + layer_num, idx)
    return ((u * 2.0 - 1.0) * bound).reshape(in_channels, out_channels)


def init_weight_shard(in_channels: int, out_channels: int, layer_num: int, seed: Optional[int],
                      row0: int, col0: int, local_cols: int, flat_start: int, flat_count: int,
                      device) -> torch.Tensor:
    """``flat_count`` entries, starting at ``flat_start``, of the row-major local block
    ``[.., local_cols]`` whose corner is ``(row0, col0)`` of the zero-padded weight matrix.

    Only the shard is ever materialised (on the device by one kernel); the reference draws the
    full matrix on every rank and slices it (plexus/gcn_conv.py:332-390).
    """
    device = torch.device(device)
    bound = 1.0 / math.sqrt(in_channels) if in_channels > 0 else 0.0
    if device.type == "cuda":
        from ..ops import _ext
        from ..ops import cuda as opc

        out = torch.empty(flat_count, dtype=torch.float32, device=device)
        _ext.load().weight_init_shard(out, flat_start, local_cols, row0, col0, in_channels, out_channels,
                                      _weight_seed(seed), WEIGHT_STREAM + layer_num, bound)
        opc._count(1)
        return out
    from ..data.synthetic import uniform01

    f = torch.arange(flat_start, flat_start + flat_count, dtype=torch.int64)
    r, c = row0 + f // local_cols, col0 + f % local_cols
    valid = (r < in_channels) & (c < out_channels)
    u = uniform01(_weight_seed(seed), WEIGHT_STREAM + layer_num, torch.where(valid, r * out_channels + c, 0))
    return torch.where(valid, (u * 2.0 - 1.0) * bound, torch.zeros(()))


class GCNConv(torch.nn.Module):
    """3D-parallel GCNConv layer (no bias).

    ``weight`` is a flat 1-D fp32 parameter: this rank's depth slice of its
    ``(in/inner) x (out/outer)`` block of the zero-padded weight matrix.
    """

    def __init__(self, in_channels, out_channels, layer_num, activation: Optional[str] = None,
                 seed: Optional[int] = None, device=None, order: str = "aggregate_first", **kwargs):
        """``order``: ``"aggregate_first"`` computes ``(A.H).W`` as the reference does;
        ``"combine_first"`` computes ``A.(H.W)`` (not for layer 0); ``"auto"`` picks
        combine-first when the padded output width is below the local input width."""
        super().__init__()
        self.layer_num = layer_num
        self.activation = activation
        grid = get_grid()
        roles = grid.roles(layer_num)
        self.outer_group, self.inner_group, self.depth_group = (
            roles.outer_group, roles.inner_group, roles.depth_group,
        )
        self.outer_group_size, self.inner_group_size, self.depth_group_size = (
            roles.outer_size, roles.inner_size, roles.depth_size,
        )
        self.outer_rank, self.inner_rank, self.depth_rank = (
            roles.outer_rank, roles.inner_rank, roles.depth_rank,
        )
        align = runtime.flags.channel_align
        # only the input features (layer 0) are sharded over depth
        self.gather_features = layer_num == 0
        self.true_in_channels, self.true_out_channels = in_channels, out_channels

        base_in = padded_channels(in_channels, self.inner_group_size, 1, align)
        if layer_num == 0:
            self.gather_weights = True
        else:
            self.gather_weights = (base_in // self.inner_group_size) % self.depth_group_size == 0
        if self.gather_weights:
            self.in_channels = padded_channels(in_channels, self.inner_group_size, self.depth_group_size, align)
        else:
            self.in_channels = base_in
        self.out_channels = padded_channels(out_channels, self.outer_group_size, 1, align)
        self.local_in_channels = self.in_channels // self.inner_group_size
        self.local_out_channels = self.out_channels // self.outer_group_size
        if order == "auto":
            order = (
                "combine_first"
                if layer_num > 0 and self.out_channels < self.local_in_channels
                else "aggregate_first"
            )
        if order not in ("aggregate_first", "combine_first"):
            raise ValueError("order must be 'aggregate_first', 'combine_first' or 'auto'")
        if order == "combine_first" and layer_num == 0:
            raise ValueError("combine_first is not available for layer 0 (depth-sharded input)")
        self.combine_first = order == "combine_first"
        # how the weight columns are split: over the outer axis, or not at all (combine-first)
        self.w_col_parts = 1 if self.combine_first else self.outer_group_size
        self.w_col_rank = 0 if self.combine_first else self.outer_rank
        self.local_weight_cols = self.out_channels // self.w_col_parts

        if device is None:
            from ..parallel.grid import default_device

            device = default_device()
        # this rank's flat shard is generated directly: rows by inner rank, columns by outer rank
        # (or all of them), row-major, and of that the depth rank's contiguous slice
        block_elems = self.local_in_channels * self.local_weight_cols
        if self.gather_weights:
            if block_elems % self.depth_group_size:
                raise ValueError(f"cannot split {block_elems} weight elements in {self.depth_group_size} depth slices")
            per = block_elems // self.depth_group_size
            flat_start, flat_count = self.depth_rank * per, per
        else:
            flat_start, flat_count = 0, block_elems
        flat = init_weight_shard(
            in_channels, out_channels, layer_num, seed,
            row0=self.inner_rank * self.local_in_channels, col0=self.w_col_rank * self.local_weight_cols,
            local_cols=self.local_weight_cols, flat_start=flat_start, flat_count=flat_count, device=device,
        )
        self.weight = Parameter(flat, requires_grad=True)

    def spec(self, edge_index, relu: Optional[bool] = None) -> LayerSpec:
        return LayerSpec(
            layer_num=self.layer_num,
            local_features_shape=(edge_index.shape[1], self.local_in_channels),
            local_weight_shape=(self.local_in_channels, self.local_weight_cols),
            depth_group=self.depth_group,
            outer_group=self.outer_group,
            inner_group=self.inner_group,
            gather_features=self.gather_features,
            gather_weights=self.gather_weights,
            relu=(self.activation == "relu") if relu is None else relu,
            combine_first=self.combine_first,
            local_out_channels=self.local_out_channels,
        )

    # the adjacency and the input features are expected to be sharded already
    def forward(self, x, edge_index_shards):
        edge_index, edge_index_t = edge_index_shards[self.layer_num % len(edge_index_shards)]
        s = self.spec(edge_index)
        return GCNConvFunction.apply(
            x, edge_index, edge_index_t, self.weight,
            s.local_features_shape, s.local_weight_shape,
            s.depth_group, s.outer_group, s.inner_group,
            s.gather_features, s.gather_weights, s.layer_num, s.relu,
            s.combine_first, s.local_out_channels,
        )

    def full_weight_block(self) -> torch.Tensor:
        """This rank's ``(in/inner) x (out/outer)`` block (depth-gathered), fp32."""
        w = self.weight.detach()
        if self.gather_weights:
            w = coll.all_gather(w, dim=0, process_group=self.depth_group)
        return w.reshape(self.local_in_channels, self.local_weight_cols)
