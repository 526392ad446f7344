"""Communication-time model: ranks every power-of-two grid (X, Y, Z) of G GPUs.

Per layer the model adds the ring-style costs of the collectives of a
3D-parallel GCN layer (reference: performance/comm_model.py:130-206):

=====================  ===========  ===========================  =========
collective             group        message (elements)           when
=====================  ===========  ===========================  =========
all-gather H           depth        N*D/(outer*inner)            layer 0 fwd
all-reduce AGG         outer        N*D/(depth*inner)            fwd
all-gather W           depth        D*D'/(outer*inner)           fwd, 2x bwd*
all-reduce OUT         inner        N*D'/(depth*outer)           fwd
all-reduce gradAGG     outer        N*D/(depth*inner)            bwd
reduce-scatter gradH   depth        N*D/(outer*inner)            bwd layer 0
all-reduce gradH       depth        N*D/(outer*inner)            bwd layer>0
=====================  ===========  ===========================  =========

(* the second backward weight term is the reduce-scatter of gradW, same cost.)

all-gather / reduce-scatter cost ``(p-1)/p * M / bw`` and all-reduce twice
that.  ``machine="perlmutter"`` / ``"frontier"`` with ``version`` v1/v2/v3
reproduce the reference's bandwidth tables (performance/comm_model.py:26-80)
and 4-byte elements.  ``machine="b200_nvl8"`` models one NVSwitch box and
prices the forms this package runs there (``parallel/fused.py``), with 2-byte
(bf16) elements and the link figures of ``perf/b200_links.json`` (measured;
``PLEXUS_LINK_MEASUREMENTS`` names another file): every group sees the same
per-GPU port bandwidth whatever its placement and each collective pays a
latency term;

* all-reduce on a 2-rank axis - one-shot push: M bytes per port and direction,
  then a reduce pass of 3 M bytes through HBM;
* all-reduce on a larger axis - reduced inside the switch (multimem):
  (1 + 1/p) M bytes per port and direction at the measured switch-reduce rate,
  then a copy of 2 M bytes through HBM;
* all-gather / reduce-scatter: (p-1)/p M bytes per port.
"""

from __future__ import annotations

import json
import os
from typing import Dict, Sequence, Tuple

from .common import DEPTH, INNER, OUTER, split_into_three_powers_of_two  # noqa: F401

GIB = float(1024**3)



def load_link_measurements(path: str = None) -> dict:
    """Measured NVLink / NVSwitch figures of the B200 box (``perf/b200_links.json`` by default)."""
    path = path or os.environ.get("PLEXUS_LINK_MEASUREMENTS") or os.path.join(
        os.path.dirname(os.path.abspath(__file__)), "b200_links.json")
    with open(path) as f:
        m = json.load(f)
    m["latency_us"] = {int(k): float(v) for k, v in m["latency_us"].items()}
    return m


_LINKS = load_link_measurements()
B200_PORT_GBS = float(_LINKS["port_gbs"])
B200_ALLREDUCE_BUS_GBS = float(_LINKS["allreduce_bus_gbs"])
B200_SWITCH_REDUCE_GBS = float(_LINKS["switch_reduce_port_gbs"])
B200_HBM_GBS = float(_LINKS["hbm_gbs"])
B200_LATENCY_US = _LINKS["latency_us"]


def b200_all_reduce_seconds(p: int, nbytes: float) -> float:
    """Time of one all-reduce of ``nbytes`` on a ``p``-rank axis in the form this package uses."""
    if p <= 1:
        return 0.0
    lat = B200_LATENCY_US.get(p, 12.0) * 1e-6
    if p == 2:
        return lat + nbytes / (B200_PORT_GBS * 1e9) + 3 * nbytes / (B200_HBM_GBS * 1e9)
    return lat + (1 + 1 / p) * nbytes / (B200_SWITCH_REDUCE_GBS * 1e9) + 2 * nbytes / (B200_HBM_GBS * 1e9)


def get_bw(ip, my, GPUS_PER_NODE, version, machine):
    """Bandwidth (GB/s) seen by a group of ``my`` ranks whose inner stride spans ``ip`` ranks."""
    if version == "v1":
        return 1
    if machine == "b200_nvl8":
        return 1 if my == 1 else B200_PORT_GBS
    if version == "v2":
        if machine == "perlmutter":
            return 200 if ip * my <= GPUS_PER_NODE else 100 / min(GPUS_PER_NODE, ip)
        return None
    if version == "v3":
        if machine == "perlmutter":
            if my == 1:
                return 1
            table = {1: {2: 76, 4: 225}, 2: {2: 76}}
            if ip in table and my in table[ip]:
                return table[ip][my]
            if ip == 1:
                return 66.59 if my >= 8 else None
            if ip == 2:
                return 66.59 / 2 if my >= 4 else None
            return 66.59 / 4
        if machine == "frontier":
            table = {1: {2: 129, 4: 52, 8: 135}, 2: {2: 50, 4: 72}, 4: {2: 36}}
            if ip in table and my in table[ip]:
                return table[ip][my]
            return {1: 40.0, 2: 20.0, 4: 10.0}.get(ip, 5.0)
    return None


def _ag(p, elems, bw, bytes_per):
    return (p - 1) / p * elems * (bytes_per / GIB) / bw


def _ar(p, elems, bw, bytes_per):
    return 2 * _ag(p, elems, bw, bytes_per)


def layer_collectives(i: int, N: int, D: int, D_next: int, sizes: Dict[str, int]):
    """``[(kind, axis, p, elements)]`` for layer ``i`` (forward then backward)."""
    o, n, d = OUTER[i % 3], INNER[i % 3], DEPTH[i % 3]
    po, pi, pd = sizes[o], sizes[n], sizes[d]
    h = N * D / (po * pi)
    agg = N * D / (pd * pi)
    w = D * D_next / (po * pi)
    out = N * D_next / (pd * po)
    fwd = ([("ag", d, pd, h)] if i == 0 else []) + [
        ("ar", o, po, agg), ("ag", d, pd, w), ("ar", n, pi, out),
    ]
    bwd = [("ag", d, pd, w), ("rs", d, pd, w), ("ar", o, po, agg)]
    bwd.append(("rs", d, pd, h) if i == 0 else ("ar", d, pd, h))
    return fwd + bwd


def compute_config_costs(G, N, D_list, version, machine):
    """Estimated communication time (ms) per epoch for each grid, ascending.

    Args:
        G: number of GPUs; N: number of nodes
        D_list: widths per layer, e.g. ``[100, 128, 128, 60]`` for 3 layers
        version: ``v1`` bandwidth-agnostic, ``v2`` theoretical, ``v3`` empirical
        machine: ``perlmutter``, ``frontier`` or ``b200_nvl8``
    """
    per_node = {"perlmutter": 4, "frontier": 8, "b200_nvl8": 8}[machine]
    b200 = machine == "b200_nvl8" and version != "v1"
    bytes_per = 2 if b200 else 4
    costs = {}
    for X, Y, Z in split_into_three_powers_of_two(G):
        sizes = {"X": X, "Y": Y, "Z": Z}
        # placement hierarchy: Y fastest, then X, then Z
        bw = {
            "Y": get_bw(1, Y, per_node, version, machine),
            "X": get_bw(Y, X, per_node, version, machine),
            "Z": get_bw(Y * X, Z, per_node, version, machine),
        }
        total = 0.0
        for i in range(len(D_list) - 1):
            for kind, axis, p, elems in layer_collectives(i, N, D_list[i], D_list[i + 1], sizes):
                if b200:
                    if p == 1:
                        continue
                    if kind == "ar":
                        total += b200_all_reduce_seconds(p, elems * bytes_per)
                    else:
                        lat = B200_LATENCY_US.get(p, 12.0) * 1e-6
                        total += lat + (p - 1) / p * elems * bytes_per / (B200_PORT_GBS * 1e9)
                else:
                    f = _ar if kind == "ar" else _ag
                    total += f(p, elems, bw[axis], bytes_per)
        costs[(X, Y, Z)] = total * 1000
    return dict(sorted(costs.items(), key=lambda kv: kv[1]))


def load_measured_peaks(path: str = None):
    """Measured HBM / GEMM peaks written next to the repository root, if present."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = path or os.path.join(here, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f)
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "fallback": True}
