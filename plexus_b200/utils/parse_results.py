"""Parse the timer-tree text of a training log into epoch / communication time.

The log contains one block per timed epoch (a line with ``epoch ``) followed
by region lines ``name | Max Time: .. ms | Avg Time: .. ms | ...``.  As in the
reference parser (reference: examples/parse_results.py:14-77):

* communication = sum of the ``Avg Time`` of lines naming a collective
  (``gather``, ``all-reduce``, ``reduce-scatter``);
* computation   = the five SpMM / GEMM regions;
* loss          = lines containing ``cross entropy``;
* epoch time    = communication + computation + loss (not the ``epoch`` timer).

Returns the means over epochs after dropping ``warmup`` of them.
"""

from __future__ import annotations

import re
from typing import Tuple

_AVG = re.compile(r"Avg Time: ([0-9]*\.?[0-9]+)")
COMM_KEYS = ("gather ", "all-reduce ", "reduce-scatter ")
COMP_KEYS = (
    "AGG = A * H ",
    "OUT = AGG * W ",
    "GRAD_W = AGG.T * GRAD_OUT ",
    "GRAD_AGG = GRAD_OUT * W.T ",
    "GRAD_H = A.T * GRAD_AGG ",
)
LOSS_KEYS = ("cross entropy",)


def extract_avg_time(line: str) -> float:
    m = _AVG.search(line)
    return float(m.group(1)) if m else 0


def process_log_file(filename: str, warmup: int) -> Tuple[float, float]:
    """``(mean epoch ms, mean communication ms)`` over the non-warm-up epochs."""
    epochs = []  # [comm, comp, loss] per epoch block
    cur = None
    with open(filename, "r") as f:
        for raw in f:
            line = raw.strip()
            if "epoch " in line:
                if cur is not None:
                    epochs.append(cur)
                cur = [0.0, 0.0, 0.0]
            elif cur is None:
                continue
            elif any(k in line for k in COMM_KEYS):
                cur[0] += extract_avg_time(line)
            elif any(k in line for k in COMP_KEYS):
                cur[1] += extract_avg_time(line)
            elif any(k in line for k in LOSS_KEYS):
                cur[2] += extract_avg_time(line)
    if cur is not None:
        epochs.append(cur)
    kept = epochs[warmup:]
    n = len(kept)
    return sum(sum(e) for e in kept) / n, sum(e[0] for e in kept) / n
