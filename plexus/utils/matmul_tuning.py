from plexus_b200.utils.matmul_tuning import (  # noqa: F401
    change_layouts,
    matmul,
    matmul_to_index,
    time_gpu,
    transpose_orders,
    tuned_matmul,
)
