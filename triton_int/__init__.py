"""Import-path alias: ``import triton_int`` resolves to ``triton_int_b200`` so that model code
written against the reference package (``triton_int.nn.linear.W8A8B8O8Linear``,
``triton_int.kernels.bmm.bmm_s8t_s8n_f32t`` ...) runs on this library unchanged."""
import importlib
import sys

import triton_int_b200 as _impl

_SUBMODULES = [
    "kernels", "kernels.linear", "kernels.bmm", "kernels.fused",
    "functional", "functional.bmm", "functional.fused", "functional.quantization",
    "nn", "nn.linear", "nn.bmm", "nn.fused",
]
for _name in _SUBMODULES:
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"triton_int_b200.{_name}")

kernels = sys.modules[f"{__name__}.kernels"]
functional = sys.modules[f"{__name__}.functional"]
nn = sys.modules[f"{__name__}.nn"]
config = _impl.config
