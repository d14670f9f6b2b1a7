"""int8 batched matmuls for attention.  "s8t" operands are row-major [B, rows, cols];
an "s8n" second operand is [B, N, K] (K contiguous), an "s8t" second operand is
[B, K, N].  Names and argument order follow the reference's
``triton_int/kernels/bmm.py``; inputs must be 3-D (kernels/bmm.py:131,282).
"""
from __future__ import annotations

import torch

from .. import _lib
from . import register_torch_op
from ._gemm import gemm


def _check_nt(a, b):
    assert a.dim() == 3 and b.dim() == 3
    assert a.shape[0] == b.shape[0]
    assert a.shape[2] == b.shape[2], "Incompatible dimensions"


def _check_nn(a, b):
    assert a.dim() == 3 and b.dim() == 3
    assert a.shape[0] == b.shape[0]
    assert a.shape[2] == b.shape[1], "Incompatible dimensions"


@register_torch_op("(Tensor a, Tensor b, Tensor? out=None) -> Tensor")
def bmm_s8t_s8t_s32t(a, b, out=None):
    """int32 A[B,M,K] . B[B,K,N]   -- reference kernels/bmm.py:12-160."""
    _check_nn(a, b)
    return gemm(a, b, False, torch.int32, _lib.EPI_I32, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor? out=None) -> Tensor")
def bmm_s8t_s8n_s32t(a, b, out=None):
    """int32 A[B,M,K] . B[B,N,K]^T   -- reference kernels/bmm.py:163-311."""
    _check_nt(a, b)
    return gemm(a, b, True, torch.int32, _lib.EPI_I32, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor scale, Tensor? out=None, ScalarType dtype=float, bool causal=False) -> Tensor")
def bmm_s8t_s8n_f32t(a, b, scale, out=None, dtype=torch.float32, causal=False):
    """dtype(scale * A . B^T)   -- reference kernels/bmm.py:314-464.
    ``causal=True`` (extension) leaves output tiles that lie entirely above the
    causal diagonal unwritten; a causal softmax never reads them."""
    _check_nt(a, b)
    return gemm(a, b, True, dtype, _lib.EPI_SCALE, alpha=scale, out=out, causal=causal)


@register_torch_op("(Tensor a, Tensor b, Tensor scale, Tensor? out=None) -> Tensor")
def bmm_s8t_s8n_s8t(a, b, scale, out=None):
    """int8(scale * A . B^T)   -- reference kernels/bmm.py:467-612."""
    _check_nt(a, b)
    return gemm(a, b, True, torch.int8, _lib.EPI_SCALE, alpha=scale, out=out)


@register_torch_op("(Tensor a, Tensor b, Tensor scale, Tensor? out=None) -> Tensor")
def bmm_s8t_s8t_s8t(a, b, scale, out=None):
    """int8(scale * A[B,M,K] . B[B,K,N])   -- reference kernels/bmm.py:615-760."""
    _check_nn(a, b)
    return gemm(a, b, False, torch.int8, _lib.EPI_SCALE, alpha=scale, out=out)
