"""Names of the reference's ``plexus/gcn_conv.py`` (``GCNConv``, ``GCNConvFunction``, ``extract_csr_submatrix``,
``chunked_spmm_all_reduce``); implementation: ``plexus_b200/models/gcn_conv.py``."""

from plexus_b200.models.gcn_conv import (  # noqa: F401
    GCNConv,
    GCNConvFunction,
    GCNStackFunction,
    chunked_spmm_all_reduce,
    extract_csr_submatrix,
)
