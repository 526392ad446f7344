from plexus_b200.models.gcn_conv import (  # noqa: F401
    GCNConv,
    GCNConvFunction,
    GCNStackFunction,
    chunked_spmm_all_reduce,
    extract_csr_submatrix,
)
