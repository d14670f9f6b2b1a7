"""triton_int_b200: the INT8 (W8A8, SmoothQuant-style) operator set of
``triton_int`` as hand-written CUDA for sm_100a behind the same Python interface:
``kernels`` (functional wrappers), ``functional`` (aliases and quantisation
helpers) and ``nn`` (modules).  There is no CPU path and no other backend."""
from . import config  # noqa: F401
from ._lib import device_status, launch_count, lib_path  # noqa: F401

__all__ = ["config", "device_status", "launch_count", "lib_path"]
