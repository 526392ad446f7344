"""Collectives carried out by kernels that store into / load from peer memory over NVLink.

Matrix all-reduces fused with the kernel that produces the matrix (``spmm_all_reduce`` /
``gemm_all_reduce``), by axis size and message size:

* one-shot (2-rank axes; any axis for messages up to 1 MiB): the compute kernel's epilogue writes
  every result row to the local output *and* into this rank's receive slot on each peer of the axis
  (plain 16-byte stores, overlapped with the rest of the kernel's work); a second launch publishes a
  flag, waits for the peers' flags and sums the received partials into the output in fp32, in
  group-rank order (ReLU / ReLU-derivative mask applied after the sum);
* segment reduce (larger axes, large messages): the compute kernel writes its partial into the
  axis' symmetric buffer; after a flag barrier every rank reduces its row segment inside the NVSwitch
  (``multimem.ld_reduce``), applies ReLU / the mask and writes the result to every rank
  (``multimem.st``); a flagged copy moves the buffer to the output.  In row chunks, the reduce of one
  chunk on a side stream while the next is computed (``csrc/kernels/nvls_reduce.cu``);
* two-shot by peer stores (``PLEXUS_TWO_SHOT=1``): the epilogue stores each row only where it is
  reduced (a reduce-scatter overlapped with the compute), a second launch reduces the own segment and
  stores it into every peer's receive slot of the next op, a third lands the peers' segments;
* NCCL after the compute kernel: axes that span hosts, or ``PLEXUS_SEGMENT_REDUCE=0``.

``spmm_reduce_scatter`` keeps only the reduce-scatter half.  ``all_reduce_f32`` (SUM / MAX),
``all_reduce_bf16`` and ``all_gather`` are push-copy kernel + flagged consumer, used for the
cross-entropy row statistics, weight shards and small tensors; ``reduce_grad_f32`` reduces weight
gradients on its own workspace channel and a side stream.

These replace the NCCL calls of ``parallel.collectives`` when ``init(comm="fused")`` is used
(reference call sites: plexus/gcn_conv.py:177-278, plexus/cross_entropy.py:46-98).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import backend, symm


class _Backend:
    """Kernels (``load()``) and compute ops (attribute access) bound by ``runtime.init``."""

    @staticmethod
    def load():
        return backend.C()

    def __getattr__(self, name):
        return getattr(backend.ops(), name)


opc = _Backend()

KID_SPMM, KID_GEMM, KID_GATHER, KID_BARRIER, KID_XENT = 1, 2, 3, 4, 5
KID_GRAD, KID_SMALL = 9, 10  # names in parallel/watchdog.py

# The one-shot push sends the whole partial result to every peer, (p-1) x M bytes per rank.  For
# p = 2 that is the minimum.  On larger groups a bandwidth-optimal all-reduce moves 2 (p-1)/p x M
# and the in-switch reduction (1 + 1/p) x M; measured on 1M x 256 bf16 (512 MB) messages:
#     ranks   one-shot   two-shot   segment reduce   NCCL after the compute kernel   (SpMM+AR / GEMM+AR, ms)
#       4     3.18/2.68  2.49/1.84  2.52/1.43        2.54/1.62
#       8     6.73/6.10  3.12/2.78  2.47/1.41        2.48/1.62
# so groups of more than two ranks reduce large messages with the segment form by default, and the
# two-shot form is opt-in (PLEXUS_TWO_SHOT=1).  Small messages are latency bound and always use
# the one-shot push.
ONE_SHOT_MAX_RANKS = int(os.environ.get("PLEXUS_ONE_SHOT_MAX_RANKS", "2"))
SMALL_MESSAGE_BYTES = 1 << 20
TWO_SHOT = os.environ.get("PLEXUS_TWO_SHOT", "0") != "0"
# Largest message one op carries; a larger matrix is processed in row blocks, one op each, so the
# receive slots (2 buffers x p slots per axis) stay bounded however large the activations are
# (a 55M x 86 bf16 matrix is 9.5 GB; unblocked its slots alone would take 38 GB per axis).
MAX_MESSAGE_BYTES = int(os.environ.get("PLEXUS_MAX_MESSAGE_BYTES", str(2 << 30)))
# Three receive sides exist for the one-shot all-reduce of a matrix (SpMM / GEMM epilogue pushes):
#   flagged (default): one reduce launch after the compute kernel, released by the peers' flags;
#   pipelined (PLEXUS_PIPELINE=1): no flags - the partials are pushed into sentinel-kept slots and
#       a reduce kernel recognises arrived data by itself; the matrix is cut in row chunks and the
#       reduce of chunk i runs on a side stream while chunk i + 1 is computed and pushed;
#   in-kernel (PLEXUS_IN_KERNEL_REDUCE=1): the compute kernel itself sums the sentinel-kept slots.
# Measured on 2 B200 (1M x 256 bf16, ms, SpMM+AR / GEMM+AR): flagged 1.81 / 1.10, pipelined
# 2.17 / 1.22, in-kernel 2.97 / 3.02 - the reduce is a pure streaming pass that needs a full grid of
# threads to run at HBM speed; inside the compute kernels it is starved of threads, and on a side
# stream its polling CTAs take SM slots from the compute kernel.  The flagged form stays the default.
PIPELINE = os.environ.get("PLEXUS_PIPELINE", "0") != "0"
PIPELINE_CHUNKS = int(os.environ.get("PLEXUS_PIPELINE_CHUNKS", "4"))
PIPELINE_MIN_BYTES = int(os.environ.get("PLEXUS_PIPELINE_MIN_BYTES", str(16 << 20)))
REDUCE_MAX_BLOCKS = int(os.environ.get("PLEXUS_REDUCE_MAX_BLOCKS", str(148 * 4)))
IN_KERNEL_REDUCE = os.environ.get("PLEXUS_IN_KERNEL_REDUCE", "0") != "0"
# Axes of more than two ranks, large messages: the compute kernel writes its partial into a
# symmetric buffer and a segment-reduce kernel sums it inside the NVSwitch (multimem), see
# csrc/kernels/nvls_reduce.cu.  The matrix is cut in row chunks; the reduce of chunk i runs on a
# high-priority side stream (few CTAs) while chunk i + 1 is computed.  PLEXUS_SEGMENT_REDUCE=0 goes
# back to NCCL after the compute kernel.
SEGMENT_REDUCE = os.environ.get("PLEXUS_SEGMENT_REDUCE", "1") != "0"
SEGMENT_CHUNKS = int(os.environ.get("PLEXUS_SEGMENT_CHUNKS", "2"))
SEGMENT_BLOCKS = int(os.environ.get("PLEXUS_SEGMENT_BLOCKS", "64"))
ROW_BLOCK_MULTIPLE = 128  # row blocks start on a GEMM tile boundary


def _row_blocks(rows: int, row_bytes: int):
    """Row ranges of at most ``MAX_MESSAGE_BYTES`` each, starting on multiples of ``ROW_BLOCK_MULTIPLE``."""
    m = ROW_BLOCK_MULTIPLE
    per = max(m, MAX_MESSAGE_BYTES // max(1, row_bytes) // m * m)
    if rows <= per:
        return [(0, rows)]
    n = -(-rows // per)
    step = -(-(-(-rows // n)) // m) * m
    return [(r, min(rows, r + step)) for r in range(0, rows, step)]


# how often each form carried a matrix collective (for tests and the metrics sink)
op_counts = {"one_shot": 0, "two_shot": 0, "reduce_scatter": 0, "library": 0, "row_blocked": 0, "in_kernel": 0,
             "pipelined": 0, "segment_reduce": 0, "xent_exchange": 0}


def _skip() -> bool:
    from .. import runtime

    return runtime.flags.skip_collectives


def _push_path(ax, nbytes: int) -> bool:
    # an axis that spans hosts has no peer-memory workspace: everything goes through NCCL
    return ax.same_host and (ax.p <= ONE_SHOT_MAX_RANKS or nbytes <= SMALL_MESSAGE_BYTES)


def _two_shot_path(ax, rows: int, cols: int, dtype) -> bool:
    ok = backend.emulated or (dtype == torch.bfloat16 and cols % 8 == 0)
    return ax.same_host and TWO_SHOT and ok and rows >= ax.p


def _segment(ax, rows: int):
    """Rows per owner and the row range ``[r0, r0 + n)`` of every group rank."""
    seg = (rows + ax.p - 1) // ax.p
    ranges = [(min(q * seg, rows), max(0, min(seg, rows - q * seg))) for q in range(ax.p)]
    return seg, ranges


def _two_shot_begin(ax, rows: int, cols: int, esz: int):
    """Reserve the op of the reduce-scatter half; returns what the compute kernel needs."""
    seg, ranges = _segment(ax, rows)
    ax.ensure(seg * cols * esz)
    epoch, buf = ax.next_op()
    return seg, ranges, epoch, buf


def _two_shot_finish(ax, out, seg, ranges, epoch, buf, relu, mask, kid):
    """Reduce this rank's segment and broadcast it (op ``epoch``), then land the peers' (next op)."""
    C = _Backend.load()
    st = opc.status_buffer(out.device)
    cols, esz = out.shape[1], out.element_size()
    assert out.stride(0) == cols and out.stride(1) == 1
    if mask is not None and mask.dtype != out.dtype:
        mask = mask.to(out.dtype)
    epoch2, buf2 = ax.next_op()
    remote, local = ax.sync(buf)
    r0, n = ranges[ax.rank]
    C.reduce_segment(out, r0, n, ax.recv_slots(buf), cols, bool(relu), mask, ax.push_targets(buf2),
                     remote, local, epoch, ax.timeout_ms, kid, st, ax.rank)
    remote2, local2 = ax.sync(buf2)
    base = out.data_ptr()
    C.gather_segments(ax.recv_slots(buf2), [base + ranges[q][0] * cols * esz for q in ax.peers],
                      [ranges[q][1] * cols * esz for q in ax.peers], remote2, local2, epoch2,
                      ax.timeout_ms, KID_GATHER, st)
    opc._count(2)


def _pipeline_chunks(rows: int, row_bytes: int):
    """Row ranges of the pipelined one-shot form (multiples of 128 rows)."""
    if PIPELINE_CHUNKS <= 1 or rows * row_bytes < PIPELINE_MIN_BYTES:
        return [(0, rows)]
    step = -(-(-(-rows // PIPELINE_CHUNKS)) // 128) * 128
    return [(r, min(rows, r + step)) for r in range(0, rows, step)]


class _SideStream:
    """The axis' side stream for the overlapped reduces (a no-op on the host emulation)."""

    def __init__(self, ax):
        self.on = not backend.emulated
        if self.on:
            if getattr(ax, "_side_stream", None) is None:
                # high priority: its few CTAs go first when a compute kernel is queued beside them
                ax._side_stream = torch.cuda.Stream(priority=-1)
            self.side = ax._side_stream
            self.main = torch.cuda.current_stream()

    def run(self, fn):
        """``fn`` after everything issued so far on the main stream, on the side stream."""
        if not self.on:
            return fn()
        self.side.wait_stream(self.main)
        with torch.cuda.stream(self.side):
            return fn()

    def join(self):
        if self.on:
            self.main.wait_stream(self.side)


def _segment_path(ax, rows: int, cols: int, dtype) -> bool:
    ok = backend.emulated or (dtype == torch.bfloat16 and cols % 8 == 0)
    # fewer rows than ranks is fine: a rank whose segment is empty only takes part in the barriers
    return ax.same_host and SEGMENT_REDUCE and not TWO_SHOT and ok and rows >= 1


def _segment_chunks(rows: int, row_bytes: int):
    if SEGMENT_CHUNKS <= 1 or rows * row_bytes < PIPELINE_MIN_BYTES:
        return [(0, rows)]
    step = -(-(-(-rows // SEGMENT_CHUNKS)) // 128) * 128
    return [(r, min(rows, r + step)) for r in range(0, rows, step)]


def _segment_all_reduce(ax, rows: int, cols: int, like: torch.Tensor, compute, relu, mask, kid):
    """All-reduce through the axis' symmetric buffer.  ``compute(r0, r1, dst)`` writes the partial
    rows ``[r0, r1)`` into ``dst`` (a view of the buffer).  Rows are blocked so that the buffer
    never exceeds ``MAX_MESSAGE_BYTES``."""
    C = _Backend.load()
    st = opc.status_buffer(like.device)
    esz = like.element_size()
    out = torch.empty((rows, cols), dtype=like.dtype, device=like.device)
    if mask is not None and mask.dtype != like.dtype:
        mask = mask.to(like.dtype)
    blocks = _row_blocks(rows, cols * esz)
    if len(blocks) > 1:
        op_counts["row_blocked"] += 1
    ax.ensure_symmetric(max(b1 - b0 for b0, b1 in blocks) * cols * esz)
    side = _SideStream(ax)
    for b0, b1 in blocks:
        S = ax.symmetric_view(b1 - b0, cols, like.dtype)
        for c0, c1 in _segment_chunks(b1 - b0, cols * esz):
            compute(b0 + c0, b0 + c1, S[c0:c1])

            def finish(c0=c0, c1=c1):
                _seg, ranges = _segment(ax, c1 - c0)
                s0, n = ranges[ax.rank]
                epoch, buf = ax.next_op()
                remote, local = ax.sync(buf)
                if n:
                    seg_mask = None if mask is None else mask[b0 + c0 + s0 : b0 + c0 + s0 + n]
                    C.segment_reduce(ax.sym_mc, ax.sym_ptrs, ax.rank, S[c0 + s0 : c0 + s0 + n], bool(relu), seg_mask,
                                     remote, local, epoch, ax.timeout_ms, kid, st, SEGMENT_BLOCKS)
                else:  # more ranks than rows in this chunk: take part in the barrier only
                    C.gather_segments([], [], [], remote, local, epoch, ax.timeout_ms, kid, st)
                epoch2, buf2 = ax.next_op()
                remote2, local2 = ax.sync(buf2)
                dst = out[b0 + c0 : b0 + c1]
                C.gather_segments([S[c0:c1].data_ptr()], [dst.data_ptr()], [(c1 - c0) * cols * esz], remote2, local2,
                                  epoch2, ax.timeout_ms, KID_GATHER, st)
                opc._count(2)

            side.run(finish)
        # the next row block reuses the buffer: everything of this one must have been copied out
        side.join()
    op_counts["segment_reduce"] += 1
    return out


def _reduce_sentinel(ax, out, slots, slot_ld, relu, mask, kid):
    _Backend.load().reduce_sentinel(out, slots, slot_ld, bool(relu), mask, ax.timeout_ms, kid,
                                    opc.status_buffer(out.device), ax.rank, REDUCE_MAX_BLOCKS)
    opc._count(1)


def _sentinel_ok(dtype, cols: int) -> bool:
    return backend.emulated or (dtype == torch.bfloat16 and cols % 8 == 0)


def _reduce(ax, out, buf, epoch, relu, mask, kid):
    remote, local = ax.sync(buf)
    _Backend.load().reduce_slots(out, ax.recv_slots(buf), out.stride(0), bool(relu), mask, remote, local,
                             epoch, ax.timeout_ms, kid, opc.status_buffer(out.device), ax.rank)
    opc._count(1)


def spmm_all_reduce(A, H, group, relu_mask=None):
    """``all_reduce_sum(A @ H)`` over ``group`` with the push fused in the SpMM epilogue."""
    if _skip():
        out = opc.spmm(A, H)
        return out if relu_mask is None else opc.relu_backward(out, relu_mask)
    ax = symm.axis_for(group)
    rows, D = A.shape[0], H.shape[1]
    if not _push_path(ax, rows * D * H.element_size()):
        if _segment_path(ax, rows, D, H.dtype):
            return _segment_all_reduce(ax, rows, D, H,
                                       lambda r0, r1, dst: opc.spmm(A, H, row_range=(r0, r1), out=dst),
                                       False, relu_mask, KID_SPMM)
        if _two_shot_path(ax, rows, D, H.dtype):
            seg, ranges, epoch, buf = _two_shot_begin(ax, rows, D, H.element_size())
            out = opc.spmm(A, H, push_ptrs=ax.push_targets(buf), push_ld=D, push_seg=(seg, ax.rank))
            _two_shot_finish(ax, out, seg, ranges, epoch, buf, False, relu_mask, KID_SPMM)
            op_counts["two_shot"] += 1
            return out
        op_counts["library"] += 1
        out = opc.spmm(A, H)
        dist.all_reduce(out, group=group)
        return out if relu_mask is None else opc.relu_backward(out, relu_mask)
    blocks = _row_blocks(rows, D * H.element_size())
    if relu_mask is not None and relu_mask.dtype != H.dtype:
        relu_mask = relu_mask.to(H.dtype)
    in_kernel = IN_KERNEL_REDUCE and opc.spmm_supports_tile_reduce(A, H)
    if PIPELINE and not in_kernel and len(blocks) == 1 and _sentinel_ok(H.dtype, D):
        esz = H.element_size()
        ax.ensure(sentinel_bytes=rows * D * esz)
        _epoch, buf = ax.next_op()
        out = torch.empty((rows, D), dtype=H.dtype, device=H.device)
        targets, slots = ax.spush_targets(buf), ax.tile_reduce(buf)[0]
        side = _SideStream(ax)
        for r0, r1 in _pipeline_chunks(rows, D * esz):
            off = r0 * D * esz
            opc.spmm(A, H, row_range=(r0, r1), out=out[r0:r1], push_ptrs=[t + off for t in targets], push_ld=D)
            side.run(lambda: _reduce_sentinel(ax, out[r0:r1], [p + off for p in slots], D, False,
                                              None if relu_mask is None else relu_mask[r0:r1], KID_SPMM))
        side.join()
        op_counts["one_shot"] += 1
        op_counts["pipelined"] += 1
        return out
    if len(blocks) == 1:
        nbytes = rows * D * H.element_size()
        ax.ensure(sentinel_bytes=nbytes) if in_kernel else ax.ensure(nbytes)
        epoch, buf = ax.next_op()
        if in_kernel:
            out = opc.spmm(A, H, relu_mask=relu_mask, push_ptrs=ax.spush_targets(buf), push_ld=D,
                           tile_reduce=ax.tile_reduce(buf))
        else:
            out = opc.spmm(A, H, push_ptrs=ax.push_targets(buf), push_ld=D)
            _reduce(ax, out, buf, epoch, False, relu_mask, KID_SPMM)
    else:
        # one op per row block: the receive slots stay bounded
        op_counts["row_blocked"] += 1
        out = torch.empty((rows, D), dtype=H.dtype, device=H.device)
        nbytes = max(r1 - r0 for r0, r1 in blocks) * D * H.element_size()
        ax.ensure(sentinel_bytes=nbytes) if in_kernel else ax.ensure(nbytes)
        for r0, r1 in blocks:
            epoch, buf = ax.next_op()
            mask_blk = None if relu_mask is None else relu_mask[r0:r1]
            if in_kernel:
                opc.spmm(A, H, relu_mask=mask_blk, row_range=(r0, r1), out=out[r0:r1],
                         push_ptrs=ax.spush_targets(buf), push_ld=D, tile_reduce=ax.tile_reduce(buf))
            else:
                opc.spmm(A, H, row_range=(r0, r1), out=out[r0:r1], push_ptrs=ax.push_targets(buf), push_ld=D)
                _reduce(ax, out[r0:r1], buf, epoch, False, mask_blk, KID_SPMM)
    op_counts["one_shot"] += 1
    if in_kernel:
        op_counts["in_kernel"] += 1
    return out


def spmm_reduce_scatter(A, H, group, relu_mask=None):
    """This rank's row segment of ``sum over ranks (A @ H)``, or ``None`` if the peer-memory path does
    not apply (rows not divisible by the group, axis across hosts, large message on a big axis).

    The SpMM epilogue stores each row only where it is reduced (own rows locally, the others into
    the owner's receive slot) and one flagged kernel sums the own segment: half the link traffic
    and a third of the reduce traffic of the all-reduce.  Used for the gradient of the
    depth-sharded input features (reference: the reduce-scatter at plexus/gcn_conv.py:268-274).
    """
    if _skip():
        return None  # the caller's all-reduce path computes without communicating
    ax = symm.axis_for(group)
    rows, D = A.shape[0], H.shape[1]
    nbytes = rows * D * H.element_size()
    if rows % ax.p or not ax.same_host:
        return None
    if not (ax.p <= ONE_SHOT_MAX_RANKS or nbytes <= SMALL_MESSAGE_BYTES or TWO_SHOT):
        return None
    if not (backend.emulated or (H.dtype == torch.bfloat16 and D % 8 == 0)):
        return None
    seg, ranges, epoch, buf = _two_shot_begin(ax, rows, D, H.element_size())
    out = opc.spmm(A, H, push_ptrs=ax.push_targets(buf), push_ld=D, push_seg=(seg, ax.rank))
    if relu_mask is not None and relu_mask.dtype != out.dtype:
        relu_mask = relu_mask.to(out.dtype)
    remote, local = ax.sync(buf)
    r0, n = ranges[ax.rank]
    _Backend.load().reduce_segment(out, r0, n, ax.recv_slots(buf), D, False, relu_mask, [], remote, local,
                                   epoch, ax.timeout_ms, KID_SPMM, opc.status_buffer(out.device), ax.rank)
    opc._count(1)
    op_counts["reduce_scatter"] += 1
    return out[r0 : r0 + n]


def gemm_all_reduce(a, W, group, relu=False, trans_b=False):
    """``act(all_reduce_sum(a @ op(W)))`` with the push fused in the tcgen05 GEMM epilogue."""
    if _skip():
        return opc.gemm(a, W, trans_b=trans_b, relu=relu)
    ax = symm.axis_for(group)
    rows = a.shape[0]
    N = W.shape[0] if trans_b else W.shape[1]
    if not _push_path(ax, rows * N * a.element_size()):
        if _segment_path(ax, rows, N, a.dtype):
            return _segment_all_reduce(ax, rows, N, a,
                                       lambda r0, r1, dst: opc.gemm(a[r0:r1], W, trans_b=trans_b, relu=False,
                                                                    out=dst),
                                       relu, None, KID_GEMM)
        if _two_shot_path(ax, rows, N, a.dtype):
            seg, ranges, epoch, buf = _two_shot_begin(ax, rows, N, a.element_size())
            out = opc.gemm(a, W, trans_b=trans_b, relu=False, push_ptrs=ax.push_targets(buf), push_ld=N,
                           push_seg=(seg, ax.rank))
            _two_shot_finish(ax, out, seg, ranges, epoch, buf, relu, None, KID_GEMM)
            op_counts["two_shot"] += 1
            return out
        op_counts["library"] += 1
        out = opc.gemm(a, W, trans_b=trans_b, relu=False)
        dist.all_reduce(out, group=group)
        return torch.relu_(out) if relu else out
    blocks = _row_blocks(rows, N * a.element_size())
    in_kernel = IN_KERNEL_REDUCE and (backend.emulated or (a.dtype == torch.bfloat16 and N % 8 == 0))
    if PIPELINE and not in_kernel and len(blocks) == 1 and _sentinel_ok(a.dtype, N):
        esz = a.element_size()
        ax.ensure(sentinel_bytes=rows * N * esz)
        _epoch, buf = ax.next_op()
        out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
        targets, slots = ax.spush_targets(buf), ax.tile_reduce(buf)[0]
        side = _SideStream(ax)
        for r0, r1 in _pipeline_chunks(rows, N * esz):
            off = r0 * N * esz
            opc.gemm(a[r0:r1], W, trans_b=trans_b, relu=False, push_ptrs=[t + off for t in targets], push_ld=N,
                     out=out[r0:r1])
            side.run(lambda: _reduce_sentinel(ax, out[r0:r1], [p + off for p in slots], N, relu, None, KID_GEMM))
        side.join()
        op_counts["one_shot"] += 1
        op_counts["pipelined"] += 1
        return out
    if len(blocks) == 1:
        nbytes = rows * N * a.element_size()
        ax.ensure(sentinel_bytes=nbytes) if in_kernel else ax.ensure(nbytes)
        epoch, buf = ax.next_op()
        if in_kernel:
            out = opc.gemm(a, W, trans_b=trans_b, relu=relu, push_ptrs=ax.spush_targets(buf), push_ld=N,
                           tile_reduce=ax.tile_reduce(buf))
        else:
            out = opc.gemm(a, W, trans_b=trans_b, relu=False, push_ptrs=ax.push_targets(buf), push_ld=N)
            _reduce(ax, out, buf, epoch, relu, None, KID_GEMM)
    else:
        op_counts["row_blocked"] += 1
        out = torch.empty((rows, N), dtype=a.dtype, device=a.device)
        nbytes = max(r1 - r0 for r0, r1 in blocks) * N * a.element_size()
        ax.ensure(sentinel_bytes=nbytes) if in_kernel else ax.ensure(nbytes)
        for r0, r1 in blocks:
            epoch, buf = ax.next_op()
            if in_kernel:
                opc.gemm(a[r0:r1], W, trans_b=trans_b, relu=relu, push_ptrs=ax.spush_targets(buf), push_ld=N,
                         out=out[r0:r1], tile_reduce=ax.tile_reduce(buf))
            else:
                opc.gemm(a[r0:r1], W, trans_b=trans_b, relu=False, push_ptrs=ax.push_targets(buf), push_ld=N,
                         out=out[r0:r1])
                _reduce(ax, out[r0:r1], buf, epoch, relu, None, KID_GEMM)
    op_counts["one_shot"] += 1
    if in_kernel:
        op_counts["in_kernel"] += 1
    return out


def all_reduce_f32(t: torch.Tensor, group, op=None) -> torch.Tensor:
    """In-place SUM or MAX all-reduce of a contiguous fp32 tensor."""
    if op in (None, dist.ReduceOp.SUM):
        code = 0
    elif op == dist.ReduceOp.MAX:
        code = 1
    else:
        raise NotImplementedError("fused all-reduce supports SUM and MAX")
    assert (t.dtype == torch.float32 or backend.emulated) and t.is_contiguous()
    if t.numel() == 0:
        return t
    ax = symm.axis_for(group)
    C = _Backend.load()
    if not _push_path(ax, t.numel() * 4):
        dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=group)
        return t
    ax.ensure(t.numel() * 4)
    epoch, buf = ax.next_op()
    C.push_copy(t, ax.push_targets(buf))
    remote, local = ax.sync(buf)
    C.reduce_slots_f32(t.view(-1), ax.recv_slots(buf), code, remote, local, epoch, ax.timeout_ms,
                       KID_SMALL, opc.status_buffer(t.device), ax.rank)
    opc._count(2)
    return t


# Cross-entropy over sharded classes with the exchange of the row statistics inside the two
# kernels (PLEXUS_XENT_EXCHANGE=1): xent_stats pushes the pairs, xent_combine starts with the flag
# barrier and reads them from the receive slots - 2 launches instead of 4.  Off by default: built
# and checked on the host emulation only, it has not run on GPUs yet.
XENT_EXCHANGE = os.environ.get("PLEXUS_XENT_EXCHANGE", "0") != "0"


def xent_exchange_combine(logits, target, class_offset, num_classes, row_offset, num_nodes, weight, group):
    """``(stats [2, R] over all class shards, loss terms of the local targets)`` for class-sharded logits,
    or ``None`` if the axis has no peer-memory workspace.  Reference: the three class-axis all-reduces
    at plexus/cross_entropy.py:46-92."""
    ax = symm.axis_for(group)
    if not ax.same_host:
        return None
    R = logits.shape[0]
    ax.ensure(2 * R * 8)  # a pair buffer is [2, R] floats (doubles on the fp64 host emulation)
    epoch, buf = ax.next_op()
    own, _ = opc.xent_stats(logits, class_offset, num_classes, push_ptrs=ax.push_targets(buf))
    remote, local = ax.sync(buf)
    ptrs = [own.data_ptr() if q == ax.rank else ax.slot(ax.rank, buf, q) for q in range(ax.p)]
    op_counts["xent_exchange"] += 1
    return opc.xent_combine_ptrs(logits, target, ptrs, row_offset, class_offset, num_nodes, weight,
                                 sync=(remote, local, epoch, ax.timeout_ms), like=own)


GRAD_CHANNEL = 1
_grad_stream = None


def reduce_grad_f32(t: torch.Tensor, group, scatter: bool, overlap: bool = True):
    """Sum a contiguous fp32 gradient over ``group``; with ``scatter`` return this rank's 1/p slice
    along dim 0 (a view of ``t``), else ``t`` reduced in place.  Returns ``(result, join)``: call
    ``join()`` before the result is used.

    The reduction has its own workspace channel and, with ``overlap``, runs on a side stream, so the
    kernels of the rest of the layer's backward - which use the same axis on the main stream - are
    not held up by it (reference: the asynchronous reduce-scatter at plexus/gcn_conv.py:242-252).
    The reduce-scatter is direct: each peer gets only the segment it owns ((p-1)/p of the tensor
    leaves this rank once), then one flagged kernel sums the own segment in place.
    """
    global _grad_stream
    ax = symm.axis_for(group, GRAD_CHANNEL)
    C = _Backend.load()
    p, n = ax.p, t.numel()
    assert t.is_contiguous() and (t.dtype == torch.float32 or backend.emulated)
    if scatter and t.shape[0] % p:
        raise ValueError(f"reduce_scatter: leading size {t.shape[0]} not divisible by {p}")
    esz = t.element_size()
    use_side = overlap and not backend.emulated
    if use_side:
        if _grad_stream is None:
            _grad_stream = torch.cuda.Stream(priority=-1)
        main = torch.cuda.current_stream()
        _grad_stream.wait_stream(main)
        ctx = torch.cuda.stream(_grad_stream)
    else:
        import contextlib

        ctx = contextlib.nullcontext()
    with ctx:
        st = opc.status_buffer(t.device)
        flat = t.view(-1)
        if scatter:
            seg = n // p
            ax.ensure(seg * esz)
            epoch, buf = ax.next_op()
            for q in ax.peers:
                C.push_copy(flat[q * seg : (q + 1) * seg], [ax.slot(q, buf, ax.rank)])
            own = flat[ax.rank * seg : (ax.rank + 1) * seg]
            remote, local = ax.sync(buf)
            C.reduce_slots_f32(own, ax.recv_slots(buf), 0, remote, local, epoch, ax.timeout_ms, KID_GRAD, st,
                               ax.rank)
            opc._count(p)
            result = t[ax.rank * (t.shape[0] // p) : (ax.rank + 1) * (t.shape[0] // p)]
        else:
            ax.ensure(n * esz)
            epoch, buf = ax.next_op()
            C.push_copy(flat, ax.push_targets(buf))
            remote, local = ax.sync(buf)
            C.reduce_slots_f32(flat, ax.recv_slots(buf), 0, remote, local, epoch, ax.timeout_ms, KID_GRAD, st,
                               ax.rank)
            opc._count(2)
            result = t
    if use_side:
        side = _grad_stream

        def join(_keep=t):
            torch.cuda.current_stream().wait_stream(side)
    else:
        def join():
            return None
    return result, join


def all_gather(t: torch.Tensor, group) -> torch.Tensor:
    """Concatenate every rank's contiguous ``t`` along dim 0 (group-rank order)."""
    ax = symm.axis_for(group)
    C = _Backend.load()
    t = t.contiguous()
    nbytes = t.numel() * t.element_size()
    if nbytes % 4:
        raise NotImplementedError("fused all-gather needs a multiple of 4 bytes per rank")
    out = torch.empty((ax.p * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    if nbytes == 0:
        return out
    if not ax.same_host:
        dist.all_gather_into_tensor(out, t, group=group)
        return out
    base = out.data_ptr()
    st = opc.status_buffer(t.device)
    # pieces of at most MAX_MESSAGE_BYTES (16-byte multiples), one op each: bounded receive slots
    piece = max(16, MAX_MESSAGE_BYTES // 16 * 16)
    ax.ensure(min(nbytes, piece))
    flat = t.view(-1)
    esz = t.element_size()
    for off in range(0, nbytes, piece):
        n = min(piece, nbytes - off)
        epoch, buf = ax.next_op()
        src = flat[off // esz : (off + n) // esz]
        C.push_copy(src, ax.push_targets(buf) + [base + ax.rank * nbytes + off])
        remote, local = ax.sync(buf)
        C.gather_slots(ax.recv_slots(buf), [base + q * nbytes + off for q in ax.peers], n, remote, local,
                       epoch, ax.timeout_ms, KID_GATHER, st)
        opc._count(2)
    return out


def all_reduce_bf16(t: torch.Tensor, group) -> torch.Tensor:
    """In-place SUM all-reduce of a contiguous bf16 matrix whose width is a multiple of 8."""
    assert (t.dtype == torch.bfloat16 or backend.emulated) and t.is_contiguous()
    t2 = t.view(-1, t.shape[-1]) if t.dim() > 1 else t.view(1, -1)
    if t2.numel() == 0:
        return t
    ax = symm.axis_for(group)
    if not _push_path(ax, t2.numel() * 2):
        if _segment_path(ax, t2.shape[0], t2.shape[1], t2.dtype):
            res = _segment_all_reduce(ax, t2.shape[0], t2.shape[1], t2,
                                      lambda r0, r1, dst: dst.copy_(t2[r0:r1]), False, None, KID_BARRIER)
            t2.copy_(res)
            return t
        if _two_shot_path(ax, t2.shape[0], t2.shape[1], t2.dtype):
            # stand-alone two-shot: scatter the rows to their owners with a copy kernel per peer
            seg, ranges, epoch, buf = _two_shot_begin(ax, t2.shape[0], t2.shape[1], 2)
            C = _Backend.load()
            for q in ax.peers:
                r0, n = ranges[q]
                if n:
                    C.push_copy(t2[r0 : r0 + n], [ax.slot(q, buf, ax.rank)])
                    opc._count(1)
            _two_shot_finish(ax, t2, seg, ranges, epoch, buf, False, None, KID_BARRIER)
            return t
        dist.all_reduce(t, group=group)
        return t
    ax.ensure(t2.numel() * 2)
    epoch, buf = ax.next_op()
    _Backend.load().push_copy(t2, ax.push_targets(buf))
    opc._count(1)
    _reduce(ax, t2, buf, epoch, False, None, KID_BARRIER)
    return t


def supports(t: torch.Tensor) -> bool:
    """Whether ``t`` can go through the peer-memory all-reduce."""
    if backend.emulated:
        return t.is_contiguous() and t.is_floating_point()
    if not t.is_cuda or not t.is_contiguous():
        return False
    if t.dtype == torch.float32:
        return True
    return t.dtype == torch.bfloat16 and t.dim() >= 1 and t.shape[-1] % 8 == 0
