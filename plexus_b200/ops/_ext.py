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


def available() -> bool:
    return os.path.exists(so_path())


def load():
    global _mod
    if _mod is None:
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        if not available():
            raise RuntimeError(
                "plexus_b200/_C.so is missing: build it with `python -m plexus_b200.build_ext` "
                "(needs nvcc; no GPU required)"
            )
        _mod = importlib.import_module("plexus_b200._C")
    return _mod
