"""Runs the UNMODIFIED reference kernels on CPU under Triton's interpreter.

TEST INFRASTRUCTURE ONLY.  This module is the "real reference" arm of the
oracle: it imports the reference package from a checkout given by the
``TRITON_INT_REFERENCE`` environment variable (a path that exists only on the
development container) and executes its ``@triton.jit`` kernels with
``TRITON_INTERPRET=1``.  It is used by ``tests/golden/make_golden.py`` to
produce the committed golden vectors and by nothing that ships.

Three harness-side shims are applied; none edits a reference file:

1. every ``triton.runtime.autotuner.Autotuner`` found in the imported kernel
   modules is pinned to its first config, because with several configs the
   autotuner benchmarks on a GPU driver, which a CPU host does not have.  The
   integer accumulation and the element-wise epilogues do not depend on the
   tile shape, so the results are unchanged;
2. ``triton_int.kernels.register_torch_op`` (kernels/__init__.py:7-24) is
   wrapped so that a schema it cannot express (the ``-> tuple`` annotation at
   kernels/fused.py:819) does not abort the import of kernels/fused.py;
3. ``tl.math.tanh`` (used at kernels/fused.py:67, removed from recent Triton)
   is supplied as ``numpy.tanh`` over the interpreter's tensor handle.
"""
from __future__ import annotations

import os
import sys

_REF = None


def reference_root():
    """Directory of the reference checkout, named by the TRITON_INT_REFERENCE environment variable."""
    return os.environ.get("TRITON_INT_REFERENCE", "")


def available() -> bool:
    root = reference_root()
    return bool(root) and os.path.isdir(os.path.join(root, "triton_int", "kernels"))


def load():
    """Import the reference under the interpreter and return a namespace of its modules."""
    global _REF
    if _REF is not None:
        return _REF
    if not available():
        raise RuntimeError("reference checkout not present (set TRITON_INT_REFERENCE)")
    if "triton" in sys.modules and os.environ.get("TRITON_INTERPRET") != "1":
        raise RuntimeError("triton was imported before TRITON_INTERPRET=1 was set")
    os.environ["TRITON_INTERPRET"] = "1"
    root = reference_root()
    if root not in sys.path:
        sys.path.insert(0, root)

    import numpy as np
    import triton
    import triton.language as tl
    from triton.runtime.autotuner import Autotuner
    from triton.runtime.interpreter import TensorHandle

    # shim 3: tl.math.tanh
    if not hasattr(tl.math, "tanh"):
        def _tanh(x, _semantic=None, _builder=None):
            h = x.handle
            return tl.tensor(TensorHandle(np.tanh(h.data), h.dtype), x.type)
        tl.math.tanh = _tanh

    # shim 2: tolerant op registration
    import triton_int.kernels as rk
    _orig = rk.register_torch_op

    def _tolerant(func):
        try:
            return _orig(func)
        except Exception:
            return func
    rk.register_torch_op = _tolerant

    import triton_int.kernels.linear as r_linear
    import triton_int.kernels.bmm as r_bmm
    import triton_int.kernels.fused as r_fused
    import triton_int.functional.fused as r_ffused
    import triton_int.functional.quantization as r_quant

    # shim 1: pin autotuners
    for mod in (r_linear, r_bmm, r_fused):
        for name in dir(mod):
            obj = getattr(mod, name)
            if isinstance(obj, Autotuner):
                obj.configs = [obj.configs[0]]

    class NS:
        pass
    ns = NS()
    ns.linear, ns.bmm, ns.fused = r_linear, r_bmm, r_fused
    ns.ffused, ns.quant = r_ffused, r_quant
    _REF = ns
    return ns
