"""``from plexus import plexus as plx; plx.init(...)`` — see plexus_b200.runtime.init.

The three feature flags stay readable as module attributes after ``init``.
"""

from plexus_b200 import runtime as _rt

block_agg = False
overlap_agg = False
tune_gemm = False


def init(*args, **kwargs):
    global block_agg, overlap_agg, tune_gemm
    grid = _rt.init(*args, **kwargs)
    block_agg, overlap_agg, tune_gemm = _rt.flags.block_agg, _rt.flags.overlap_agg, _rt.flags.tune_gemm
    return grid


init.__doc__ = _rt.init.__doc__
