"""Locate and load the compiled sm_100a extension ``plexus_b200/_C.so``.

The shared object is built in-tree by ``python -m plexus_b200.build_ext``.
There is no silent fallback: asking for the extension when it cannot be
loaded raises, so a machine with a GPU never runs a non-native path unnoticed.
"""

from __future__ import annotations

import importlib
import os

_mod = None


def so_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so")


def disabled() -> bool:
    """``PLEXUS_DISABLE_NATIVE=1`` keeps the extension out of the process: the start-up data ops
    then run as plain torch ops (on whatever device their tensors live on) and any attempt to
    launch one of the package's kernels raises.  Used by tools that must not map ``_C.so``, such
    as the baseline arm of ``bench.py`` while it builds its input shards."""
    return os.environ.get("PLEXUS_DISABLE_NATIVE", "0") not in ("", "0")


def available() -> bool:
    return not disabled() and os.path.exists(so_path())


def load():
    global _mod
    if _mod is None:
        if disabled():
            raise RuntimeError("plexus_b200's native extension is disabled in this process "
                               "(PLEXUS_DISABLE_NATIVE is set)")
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        if not available():
            raise RuntimeError(
                "plexus_b200/_C.so is missing: build it with `python -m plexus_b200.build_ext` "
                "(needs nvcc; no GPU required)"
            )
        _mod = importlib.import_module("plexus_b200._C")
    return _mod
