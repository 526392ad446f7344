from plexus_b200.models.cross_entropy import (  # noqa: F401
    TensorParallelCrossEntropy,
    parallel_accuracy,
    parallel_cross_entropy,
)
