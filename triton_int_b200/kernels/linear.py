"""W8A8 linear operators: C[..., N] = epilogue(A[..., K] . W[N, K]^T).

Same names, positional order and defaults as the reference's
``triton_int/kernels/linear.py``; each wrapper flattens the leading dimensions of
``a`` (kernels/linear.py:259-260), launches ``ti_gemm_i8`` on the current CUDA
stream and returns a view with the leading dimensions restored (:288).  ``out=``
is honoured (the reference accepts the argument but fails when it is given).
"""
from __future__ import annotations

import torch

from .. import _lib
from . import register_torch_op
from ._gemm import gemm


def _flatten(a, b):
    assert b.dim() == 2, "weight must be [N, K]"
    assert a.shape[-1] == b.shape[1], "Incompatible dimensions"
    lead = a.shape[:-1]
    a2 = a.reshape(-1, a.shape[-1])  # a view whenever the reference's .view would succeed
    return lead, a2.unsqueeze(0), b.unsqueeze(0)


def _linear(a, b, out_dtype, epilogue, bias=None, alpha=None, beta=None, out=None, residual=None):
    lead, a3, b3 = _flatten(a, b)
    c = gemm(a3, b3, True, out_dtype, epilogue, bias=bias, alpha=alpha, beta=beta, out=out, residual=residual)
    return c.view(*lead, b.shape[0])


@register_torch_op("(Tensor a, Tensor b, Tensor scale, Tensor? out=None, ScalarType dtype=float) -> Tensor")
def linear_a8_w8_ofp32(a, b, scale, out=None, dtype=torch.float):
    """dtype(scale * acc)   -- reference kernels/linear.py:24-147."""
    return _linear(a, b, dtype, _lib.EPI_SCALE, alpha=scale, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor bias, Tensor scale_a, Tensor scale_b, Tensor? out=None) -> Tensor")
def linear_a8_w8_b8_o8(a, b, bias, scale_a, scale_b, out=None):
    """int8(scale_b * bias_i8 + scale_a * acc)   -- reference kernels/linear.py:150-288."""
    return _linear(a, b, torch.int8, _lib.EPI_SCALE_BIAS, bias=bias, alpha=scale_a, beta=scale_b, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor bias, Tensor scale_a, Tensor scale_b, Tensor? out=None) -> Tensor")
def linear_relu_a8_w8_b8_o8(a, b, bias, scale_a, scale_b, out=None):
    """max(int8(...), 0)   -- reference kernels/linear.py:291-430."""
    return _linear(a, b, torch.int8, _lib.EPI_SCALE_BIAS_RELU, bias=bias, alpha=scale_a, beta=scale_b, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor? bias, Tensor? out=None) -> Tensor")
def linear_a8_w8_b32_o32(a, b, bias, out=None):
    """int32 acc + bias_i32, no scaling   -- reference kernels/linear.py:433-566.
    ``bias=None`` (raw partial sums, used by row-parallel shards) is an extension."""
    return _linear(a, b, torch.int32, _lib.EPI_I32, bias=bias, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor bias, Tensor scale_a, Tensor scale_b, Tensor? out=None) -> Tensor")
def linear_a8_w8_b32_o32_with_scaling(a, b, bias, scale_a, scale_b, out=None):
    """int32(trunc(scale_b * bias_i32 + scale_a * acc))   -- reference kernels/linear.py:569-708."""
    return _linear(a, b, torch.int32, _lib.EPI_SCALE_BIAS, bias=bias, alpha=scale_a, beta=scale_b, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor bias, Tensor scale_a, Tensor scale_b, Tensor? out=None, ScalarType? dtype=None) -> Tensor")
def linear_a8_w8_bfp32_ofp32(a, b, bias, scale_a, scale_b, out=None, dtype=None):
    """dtype(scale_b * bias + scale_a * acc); dtype defaults to the bias dtype
    -- reference kernels/linear.py:711-853 (:829-832 for the default)."""
    if dtype is None:
        dtype = out.dtype if out is not None else bias.dtype
    return _linear(a, b, dtype, _lib.EPI_SCALE_BIAS, bias=bias, alpha=scale_a, beta=scale_b, out=out)


def linear_a8_w8_b32_dq_add_ofp32(a, b, bias, dq_scale, residual, out=None):
    """fp32(residual + dq_scale * (acc + bias_i32)): a row-parallel linear whose epilogue does the
    dequantise + residual-add front half of DQ_Add_LayerNorm_Q (reference
    functional/fused.py:6-15, nn/fused.py:59-78), bit for bit what ``dq_add_layernorm_q``
    would return as its residual output; the result feeds ``layer_norm_fwd_fused_single_pass_q``.
    No counterpart kernel in the reference.  ``residual`` is fp32 with the output's shape."""
    n = b.shape[0]
    res2 = residual.reshape(-1, n)
    return _linear(a, b, torch.float32, _lib.EPI_DQ_ADD, bias=bias, alpha=dq_scale, out=out, residual=res2)
