"""The kernel library the parts call.

``get_ops()`` returns the one :class:`~torchllms_b200.kernels.native.NativeOps`
of the process: hand-written CUDA for sm_100a, compiled on first use.  There
is no other implementation in the package: without ``nvcc`` or without a GPU
the first call raises.  ``set_ops`` lets a caller that builds its own engine
pass in another object with the same methods (tests use it to run the engine's
host-side logic against plain PyTorch functions).
"""

from __future__ import annotations

from typing import Any, Optional

_ops: Optional[Any] = None


def get_ops():
    global _ops
    if _ops is None:
        from .native import NativeOps
        _ops = NativeOps()
    return _ops


def set_ops(ops) -> None:
    global _ops
    _ops = ops
