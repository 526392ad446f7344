"""Nested region timers keyed by the call stack of region names.

``start(name)`` pushes ``name`` on a stack and ``stop(name)`` pops it; the
elapsed time is accumulated under the tuple of the whole stack, so a report
can rebuild the region tree (parent key = ``key[:-1]``).  On CUDA the regions
are bracketed by CUDA events on the current stream and only resolved in
``get_times()``, so timing does not synchronize the training stream.  On CPU
``time.perf_counter`` is used.

With ``PLEXUS_NVTX=1`` (or ``Timers(nvtx=True)``) every region is also an NVTX range, whether or
not the timers are enabled, so a profiler capture can be filtered or grouped by the same region
names (the reference has no profiler hooks).

The region names used across the package are the ones the reference's log
parser matches (reference: examples/parse_results.py:46-69, plexus/gcn_conv.py
timer calls), so ``process_log_file`` works on logs of either framework.
"""

from __future__ import annotations

import os
import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch


class Timers:
    def __init__(self, enabled: bool = False, use_cuda: bool | None = None, nvtx: bool | None = None):
        self.enabled = enabled
        self._use_cuda = use_cuda
        if nvtx is None:
            nvtx = os.environ.get("PLEXUS_NVTX", "0") not in ("", "0")
        self.nvtx = bool(nvtx) and torch.cuda.is_available()
        self._stack: List[str] = []
        self._open: Dict[Tuple[str, ...], object] = {}
        self._pending: List[Tuple[Tuple[str, ...], object, object]] = []
        self._cpu_total: Dict[Tuple[str, ...], float] = defaultdict(float)
        self._count: Dict[Tuple[str, ...], int] = defaultdict(int)

    # The reference calls both ``ax.get_timers().start`` and (by mistake)
    # ``ax.get_timers.start``; making the object callable and returning itself
    # lets one instance serve both spellings.
    def __call__(self):
        return self

    @property
    def use_cuda(self) -> bool:
        if self._use_cuda is None:
            return torch.cuda.is_available()
        return self._use_cuda

    def start(self, name: str) -> None:
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if not self.enabled:
            return
        self._stack.append(name)
        key = tuple(self._stack)
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open[key] = ev
        else:
            self._open[key] = time.perf_counter()

    def stop(self, name: str) -> None:
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        if not self.enabled:
            return
        if not self._stack or self._stack[-1] != name:
            raise RuntimeError(
                f"timer stop('{name}') does not match the open region {self._stack[-1:]}"
            )
        key = tuple(self._stack)
        begin = self._open.pop(key)
        self._stack.pop()
        self._count[key] += 1
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pending.append((key, begin, ev))
        else:
            self._cpu_total[key] += (time.perf_counter() - begin) * 1e3

    def get_times(self):
        """Return ``(total_ms_by_key, count_by_key)`` and reset the totals."""
        totals: Dict[Tuple[str, ...], float] = defaultdict(float)
        if self.use_cuda and self._pending:
            torch.cuda.synchronize()
            for key, b, e in self._pending:
                totals[key] += b.elapsed_time(e)
        for key, ms in self._cpu_total.items():
            totals[key] += ms
        counts = dict(self._count)
        self._pending.clear()
        self._cpu_total.clear()
        self._count = defaultdict(int)
        return dict(totals), counts

    class _Region:
        def __init__(self, timers, name):
            self.t, self.name = timers, name

        def __enter__(self):
            self.t.start(self.name)

        def __exit__(self, *exc):
            self.t.stop(self.name)
            return False

    def region(self, name: str):
        return Timers._Region(self, name)


_TIMERS = Timers(enabled=False)


def get_timers() -> Timers:
    return _TIMERS


def configure_timers(enabled: bool, use_cuda: bool | None = None) -> Timers:
    global _TIMERS
    _TIMERS = Timers(enabled=enabled, use_cuda=use_cuda)
    return _TIMERS
