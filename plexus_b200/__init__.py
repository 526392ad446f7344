"""plexus_b200: 3D-parallel full-graph GCN training for NVIDIA B200 (sm_100a).

Public surface (the ``plexus`` package at the repository root re-exports it
under the module names of hpcgroup/plexus):

* ``init`` / ``flags``                     - grid set-up and run-time switches
* ``GCNConv``, ``GCNConvFunction``, ``Net`` - the parallel layer and model
* ``parallel_cross_entropy``               - class-sharded loss
* ``DataLoader``, ``preprocess_graph``, ``partition_graph_2d`` - data pipeline
* ``FusedAdamW``                           - multi-tensor optimizer
* ``perf``                                 - communication / compute / memory models
"""

from . import runtime
from .runtime import flags, init, shutdown, choose_grid, check_status  # noqa: F401
from .models.gcn_conv import GCNConv, GCNConvFunction, GCNStackFunction  # noqa: F401
from .models.cross_entropy import parallel_cross_entropy, parallel_accuracy  # noqa: F401
from .models.net import Net, SerialGCN  # noqa: F401
from .optim import FusedAdamW, FusedAdam  # noqa: F401
from .utils.dataloader import DataLoader  # noqa: F401
from .utils.timers import get_timers  # noqa: F401

__version__ = "0.1.0"
