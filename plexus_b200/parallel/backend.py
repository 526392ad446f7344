"""Which kernels carry the peer-memory collectives: bound once by ``runtime.init``.

On CUDA devices that is the extension (``plexus_b200._C``) and ``ops.cuda``.  For tests of the host
code on CPU ranks ``runtime.init`` binds the shared-memory emulation instead
(``parallel/emulator.py``); the collective code itself never asks which one it runs on, it only
calls ``C()`` / ``ops()`` and reads ``emulated`` where an argument check is device specific.
"""

from __future__ import annotations

from ..ops import _ext

emulated = False
_kernels = None
_ops = None


def bind(use_emulator: bool) -> None:
    global emulated, _kernels, _ops
    emulated = bool(use_emulator)
    if emulated:
        from . import emulator

        _kernels, _ops = emulator.C, emulator.ops
    else:
        _kernels, _ops = None, None  # the extension is loaded at first use


def C():
    """The kernel entry points (extension module, or its emulation)."""
    global _kernels
    if _kernels is None:
        _kernels = _ext.load()
    return _kernels


def ops():
    """The compute ops with their push epilogues (``ops.cuda``, or its emulation)."""
    global _ops
    if _ops is None:
        from ..ops import cuda

        _ops = cuda
    return _ops
