"""Process-wide settings of the operator library."""
from __future__ import annotations

import os

from . import _lib

_ROUNDING_NAMES = {"rne_sat": _lib.ROUND_RNE_SAT, "trunc_wrap": _lib.ROUND_TRUNC_WRAP}
_rounding = _ROUNDING_NAMES.get(os.environ.get("TRITON_INT_ROUNDING", "rne_sat").lower())
if _rounding is None:
    raise ValueError("TRITON_INT_ROUNDING must be 'rne_sat' or 'trunc_wrap'")
_gemm_path = {"auto": _lib.PATH_AUTO, "tcgen05": _lib.PATH_TCGEN05, "generic": _lib.PATH_GENERIC}[
    os.environ.get("TRITON_INT_GEMM_PATH", "auto").lower()]


def set_rounding_mode(name: str) -> None:
    """'rne_sat': round half to even and saturate (default).
    'trunc_wrap': truncate toward zero and keep the low byte, bit-for-bit what the
    reference kernels' ``.to(tl.int8)`` produces (kernels/linear.py:254)."""
    global _rounding
    _rounding = _ROUNDING_NAMES[name.lower()]


def rounding_mode() -> int:
    return _rounding


def rounding_mode_name() -> str:
    return {v: k for k, v in _ROUNDING_NAMES.items()}[_rounding]


def set_gemm_path(name: str) -> None:
    """'auto' (tcgen05 when the operands are tensor-map addressable, else the
    stride-agnostic kernel), 'tcgen05' (fail if not addressable) or 'generic'."""
    global _gemm_path
    _gemm_path = {"auto": _lib.PATH_AUTO, "tcgen05": _lib.PATH_TCGEN05, "generic": _lib.PATH_GENERIC}[name.lower()]


def gemm_path() -> int:
    return _gemm_path


class rounding:
    """Context manager: ``with config.rounding('trunc_wrap'): ...``"""

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        self.prev = rounding_mode_name()
        set_rounding_mode(self.name)

    def __exit__(self, *exc):
        set_rounding_mode(self.prev)
