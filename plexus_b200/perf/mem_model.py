"""Memory model: approximate GPU memory (GB) per rank for every grid.

Counted in 32-bit words, as in the reference (performance/mem_model.py:26-93):

* adjacency: for each distinct layer type, ``A`` and ``A^T`` in CSR with
  3 words per nonzero and 2 per row;
* weights: parameter + gradient + two Adam moments, sharded over all G ranks;
* AGG and activations: value + gradient;
* trainable input features: 4 copies, sharded over all ranks;
* one-time gather buffers of layer 0 and int64 labels.

``bytes_per_index`` / ``bytes_per_value`` let the same accounting describe this
framework's int32-index, bf16-activation layout (``compute_config_mem_b200``),
which also counts the peer-memory workspaces of the fused collectives
(``workspace_bytes``): per axis two buffers of p receive slots on 2-rank axes,
one symmetric buffer on larger axes, each sized by the largest message of the
axis (capped by the row-block limit ``PLEXUS_MAX_MESSAGE_BYTES``).
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


def workspace_bytes(X, Y, Z, N, D_list, max_message_bytes=2 << 30, bytes_per=2):
    """Bytes of peer-memory workspace per rank (``parallel/symm.py``) for the fused collectives.

    2-rank axis: flags + 2 buffers x p slots of the largest message (one-shot push).  Larger axis:
    one symmetric buffer of 1.25 x the largest all-reduce message (grown with headroom) plus 2 x p
    slots for the small messages and gathers (at most 1 MiB each, or the largest gathered piece).
    """
    from .comm_model import layer_collectives

    sizes = {"X": X, "Y": Y, "Z": Z}
    largest = {"X": [0.0, 0.0], "Y": [0.0, 0.0], "Z": [0.0, 0.0]}  # [all-reduce, gather / scatter]
    for i in range(len(D_list) - 1):
        for kind, axis, p, elems in layer_collectives(i, N, D_list[i], D_list[i + 1], sizes):
            if p > 1:
                k = 0 if kind == "ar" else 1
                largest[axis][k] = max(largest[axis][k], min(float(max_message_bytes), elems * bytes_per))
    total = 0.0
    for axis, (ar, ag) in largest.items():
        p = sizes[axis]
        if p == 1:
            continue
        if p == 2:
            total += 1024 + 2 * p * max(ar, ag / p)
        else:
            total += 1024 + 1.25 * ar + 2 * p * max(min(ar, 1 << 20), ag / p)
    return total


def compute_config_mem_b200(G, N, E, D_list, max_message_bytes=2 << 30, workspaces=True):
    """Same accounting for int32 indices + fp32 values (2 words/nnz, 1 word/row)
    and bf16 activations (half a word per element), plus the peer-memory workspaces."""
    out = {}
    for X, Y, Z in split_into_three_powers_of_two(G):
        gb = _words(X, Y, Z, N, E, D_list, 2.0, 1.0, 0.5) * 4 / _GB
        if workspaces:
            gb += workspace_bytes(X, Y, Z, N, D_list, max_message_bytes) / _GB
        out[f"X{X}Y{Y}Z{Z}"] = gb
    return dict(sorted(out.items(), key=lambda kv: kv[1]))
