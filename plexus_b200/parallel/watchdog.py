"""Failure detection on the host.

The reference has none: a lost rank leaves the others inside a collective
until the batch system kills the job.  Here three host-side mechanisms turn a
lost or stalled peer into an exception before (or shortly after) the next
launch, without ever faulting a device:

* :class:`Heartbeat` - every rank publishes ``(step, wall time)`` in the
  rendezvous key-value store between steps; ``check_peers`` raises
  :class:`PeerFailure` naming ranks whose beat is older than a limit or that
  announced their exit.
* :class:`EpochWatchdog` - a wall-clock deadline around each step, checked by a
  helper thread; on expiry a callback runs (by default the process exits with
  a distinct code so a launcher can restart from the last checkpoint).
* :func:`raise_on_device_status` - kernels that wait on peers give up after a
  bounded number of polls and record ``(code, kernel, peer, expected, seen)``
  in a status buffer; the host reads it after the step and raises
  :class:`PlexusCommTimeout`.
"""

from __future__ import annotations

import os
import threading
import time
from typing import Callable, List, Optional, Sequence

import torch

STATUS_OK = 0
STATUS_TIMEOUT = 1
STATUS_BOUNDS = 2
STATUS_WORDS = 8

EXIT_CODE_WATCHDOG = 43


class PlexusCommTimeout(RuntimeError):
    """A device-side wait on a peer ran out of polls."""


class PeerFailure(RuntimeError):
    """One or more peers stopped publishing heartbeats or announced exit."""

    def __init__(self, ranks: Sequence[int], reason: str):
        super().__init__(f"peer rank(s) {list(ranks)} {reason}")
        self.ranks = list(ranks)


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, prefix: str = "plexus/hb"):
        self.store, self.rank, self.world_size, self.prefix = store, rank, world_size, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def announce_exit(self, reason: str = "exit") -> None:
        self.store.set(self._key(self.rank), f"-1:{time.time():.3f}:{reason}")

    def read(self, r: int):
        """(step, timestamp) of rank ``r`` or ``None`` if it never published."""
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            raw = self.store.get(self._key(r)).decode()
        except Exception:
            return None
        parts = raw.split(":")
        return int(parts[0]), float(parts[1])

    def check_peers(self, max_age_s: float, min_step: Optional[int] = None,
                    missing_is_failure: bool = False, lag_grace_s: float = 0.0) -> None:
        """Raise :class:`PeerFailure` if a peer exited, is stale, or lags behind ``min_step``.

        Stale: the last beat is older than ``max_age_s``.  Lagging: the last published step is below
        ``min_step`` and that beat is older than ``lag_grace_s`` (a peer that still beats but is stuck
        on an old step, e.g. in a host-side loop; 0 = any peer below ``min_step`` counts).
        A peer that has not published anything yet is only a failure if ``missing_is_failure``
        (ranks reach their first beat at slightly different times).
        """
        now = time.time()
        gone, stale, lagging = [], [], []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            got = self.read(r)
            if got is None:
                if missing_is_failure:
                    stale.append(r)
                continue
            step, ts = got
            if step < 0:
                gone.append(r)
            elif now - ts > max_age_s:
                stale.append(r)
            elif min_step is not None and step < min_step and now - ts > lag_grace_s:
                lagging.append(r)
        if gone:
            raise PeerFailure(gone, "announced exit")
        if stale:
            raise PeerFailure(stale, f"sent no heartbeat for more than {max_age_s:.1f} s")
        if lagging:
            raise PeerFailure(lagging, f"still below step {min_step} after {lag_grace_s:.1f} s")

    def wait_for_peers(self, step: int, timeout_s: float, poll_s: float = 0.05) -> None:
        """Block until every peer reached ``step``; raise :class:`PeerFailure` on exit/timeout."""
        deadline = time.time() + timeout_s
        while True:
            behind, gone = [], []
            for r in range(self.world_size):
                if r == self.rank:
                    continue
                got = self.read(r)
                if got is None or (0 <= got[0] < step):
                    behind.append(r)
                elif got[0] < 0:
                    gone.append(r)
            if gone:
                raise PeerFailure(gone, "announced exit")
            if not behind:
                return
            if time.time() > deadline:
                raise PeerFailure(behind, f"did not reach step {step} within {timeout_s:.1f} s")
            time.sleep(poll_s)


class EpochWatchdog:
    """Wall-clock deadline per step, enforced by a daemon thread."""

    def __init__(self, timeout_s: float, on_timeout: Optional[Callable[[int], None]] = None,
                 poll_s: float = 0.05):
        self.timeout_s, self.poll_s = timeout_s, poll_s
        self.on_timeout = on_timeout or self._default_action
        self._deadline: Optional[float] = None
        self._step = -1
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self.fired = False
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    @staticmethod
    def _default_action(step: int) -> None:
        print(f"[plexus watchdog] step {step} exceeded its deadline; exiting", flush=True)
        os._exit(EXIT_CODE_WATCHDOG)

    def _run(self) -> None:
        while not self._stop.wait(self.poll_s):
            with self._lock:
                expired = self._deadline is not None and time.time() > self._deadline
                step = self._step
                if expired:
                    self._deadline = None
            if expired:
                self.fired = True
                self.on_timeout(step)

    def begin(self, step: int) -> None:
        with self._lock:
            self._step, self._deadline = step, time.time() + self.timeout_s

    def end(self) -> None:
        with self._lock:
            self._deadline = None

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=1.0)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


_KERNEL_NAMES = {
    1: "spmm_all_reduce", 2: "gemm_all_reduce", 3: "all_gather", 4: "barrier", 5: "xent_exchange",
    6: "gemm (mbarrier)", 7: "spmm tensor-core kernel / wait_flag probe", 8: "csr_validate",
    9: "weight_gradient_reduce", 10: "all_reduce_f32",
}


def decode_status(words: Sequence[int]) -> str:
    code, kernel, peer, expected, seen = (list(words) + [0] * 5)[:5]
    kind = {STATUS_TIMEOUT: "TIMEOUT", STATUS_BOUNDS: "BOUNDS"}.get(code, f"code {code}")
    return (
        f"{kind} in kernel '{_KERNEL_NAMES.get(kernel, kernel)}': peer/slot {peer}, "
        f"expected {expected}, seen {seen}"
    )


def raise_on_device_status(status: torch.Tensor, clear: bool = True) -> None:
    """Read a kernel status buffer (int32[STATUS_WORDS]); raise if a wait gave up."""
    host = status.detach().cpu().tolist()
    if host[0] == STATUS_OK:
        return
    if clear:
        status.zero_()
    msg = decode_status(host)
    if host[0] == STATUS_TIMEOUT:
        raise PlexusCommTimeout(msg)
    raise RuntimeError(msg)
