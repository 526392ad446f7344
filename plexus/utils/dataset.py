"""Names of the reference's ``plexus/utils/dataset.py`` (preprocessing, converters, 2-D partitioner);
implementation: ``plexus_b200/utils/dataset.py``."""

from plexus_b200.utils.dataset import (  # noqa: F401
    mtx_to_pyg,
    partition_graph_2d,
    preprocess_graph,
    print_nnz_stats,
    tsv_to_pyg,
    write_to_mtx,
)
