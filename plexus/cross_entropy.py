"""Names of the reference's ``plexus/cross_entropy.py`` (``parallel_cross_entropy``, ``TensorParallelCrossEntropy``);
implementation: ``plexus_b200/models/cross_entropy.py``."""

from plexus_b200.models.cross_entropy import (  # noqa: F401
    TensorParallelCrossEntropy,
    parallel_accuracy,
    parallel_cross_entropy,
)
