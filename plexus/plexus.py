"""``from plexus import plexus as plx; plx.init(...)`` — see plexus_b200.runtime.init.

The three feature flags stay readable as module attributes after ``init``.
"""

from plexus_b200 import runtime as _rt

block_agg = False
overlap_agg = False
tune_gemm = False


def init(G_intra_r=1, G_intra_c=1, G_intra_d=1, gpus_per_node=None, enable_internal_timers=False,
         block_aggregation=False, overlap_aggregation=False, tune_gemms=False, **kwargs):
    global block_agg, overlap_agg, tune_gemm
    grid = _rt.init(G_intra_r, G_intra_c, G_intra_d, gpus_per_node, enable_internal_timers,
                    block_aggregation, overlap_aggregation, tune_gemms, **kwargs)
    block_agg, overlap_agg, tune_gemm = _rt.flags.block_agg, _rt.flags.overlap_agg, _rt.flags.tune_gemm
    return grid


init.__doc__ = _rt.init.__doc__
