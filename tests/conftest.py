import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch

    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(skip_multi)


@pytest.fixture(autouse=True)
def _reset_runtime():
    yield
    from plexus_b200.parallel import grid
    from plexus_b200 import runtime

    grid.set_grid(None)
    runtime.flags.initialized = False
    runtime.flags.comm = "nccl"
    runtime.flags.block_agg = runtime.flags.overlap_agg = runtime.flags.tune_gemm = False
    runtime.flags.skip_collectives = False
