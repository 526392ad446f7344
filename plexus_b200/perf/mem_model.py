"""Memory model: approximate GPU memory (GB) per rank for every grid.

Counted in 32-bit words, as in the reference (performance/mem_model.py:26-93):

* adjacency: for each distinct layer type, ``A`` and ``A^T`` in CSR with
  3 words per nonzero and 2 per row;
* weights: parameter + gradient + two Adam moments, sharded over all G ranks;
* AGG and activations: value + gradient;
* trainable input features: 4 copies, sharded over all ranks;
* one-time gather buffers of layer 0 and int64 labels.

``bytes_per_index`` / ``bytes_per_value`` let the same accounting describe this
framework's int32-index, bf16-activation layout (``compute_config_mem_b200``).
"""

from __future__ import annotations

from .common import split_into_three_powers_of_two  # noqa: F401

_GB = 1024.0**3


def _words(X, Y, Z, N, E, D_list, nnz_words=3.0, row_words=2.0, act_words=1.0):
    G = X * Y * Z
    adj = 0.0
    for rows_by, cols_by in [(Z, X), (Y, Z), (X, Y)][: min(3, len(D_list))]:
        adj += 2 * (E / (rows_by * cols_by) * nnz_words + N / rows_by * row_words)
    weights = sum(4 * D_list[i] * D_list[i + 1] / G for i in range(len(D_list) - 1))
    agg_div = (Z * Y, Y * X, X * Z)
    act_div = (X * Y, Z * X, Y * Z)
    agg = sum(2 * N * D_list[i] / agg_div[i % 3] for i in range(len(D_list) - 1)) * act_words
    act = sum(2 * N * D_list[i] / act_div[i % 3] for i in range(1, len(D_list))) * act_words
    feats = 4 * N * D_list[0] / G
    one_time = (N * D_list[0]) / (X * Y) * act_words + (D_list[0] * D_list[1]) / (Y * X)
    label_div = {2: Z, 0: Y, 1: X}[len(D_list) % 3]
    labels = N * 2 / label_div
    return adj + weights + agg + act + feats + one_time + labels


def compute_config_mem(G, N, E, D_list):
    """``{"X{X}Y{Y}Z{Z}": GB}`` ascending, fp32 values and int64 indices."""
    out = {}
    for X, Y, Z in split_into_three_powers_of_two(G):
        out[f"X{X}Y{Y}Z{Z}"] = _words(X, Y, Z, N, E, D_list) * 4 / _GB
    return dict(sorted(out.items(), key=lambda kv: kv[1]))


def compute_config_mem_b200(G, N, E, D_list):
    """Same accounting for int32 indices + fp32 values (2 words/nnz, 1 word/row)
    and bf16 activations (half a word per element)."""
    out = {}
    for X, Y, Z in split_into_three_powers_of_two(G):
        out[f"X{X}Y{Y}Z{Z}"] = _words(X, Y, Z, N, E, D_list, 2.0, 1.0, 0.5) * 4 / _GB
    return dict(sorted(out.items(), key=lambda kv: kv[1]))
