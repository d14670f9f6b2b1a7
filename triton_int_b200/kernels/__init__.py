"""Host wrappers of the CUDA kernels, with the names, argument order and defaults
of the reference's ``triton_int.kernels`` package, plus the ``triton_op`` torch
library namespace the reference registers its operators under
(kernels/__init__.py:5-24)."""
from __future__ import annotations

import torch

try:
    lib = torch.library.Library("triton_op", "FRAGMENT")
except Exception:  # pragma: no cover - torch builds without the library API
    lib = None


def register_torch_op(schema: str):
    """Register ``func`` as ``torch.ops.triton_op.<name>`` for CUDA tensors with a
    full schema (the reference builds its schema from annotated parameters only,
    kernels/__init__.py:14, which leaves most of its ops uncallable through the
    dispatcher).  Returns the original function, as the reference does, so direct
    calls bypass the dispatcher."""

    def deco(func):
        if lib is not None:
            try:
                lib.define(f"{func.__name__}{schema}")
                lib.impl(func.__name__, func, "CUDA")
            except Exception:
                pass  # already defined by another import of the same namespace
        return func

    return deco
