"""Names of the reference's ``plexus/utils/matmul_tuning.py`` (``tuned_matmul`` and its helpers);
implementation: ``plexus_b200/utils/matmul_tuning.py``."""

from plexus_b200.utils.matmul_tuning import (  # noqa: F401
    change_layouts,
    matmul,
    matmul_to_index,
    time_gpu,
    transpose_orders,
    tuned_matmul,
)
