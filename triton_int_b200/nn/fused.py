"""LayerNorm-quantising and GELU-quantising modules (reference nn/fused.py)."""
from __future__ import annotations

import torch

from ..functional.fused import dq_add_layernorm_q_cpp
from ..functional.quantization import quantize_per_tensor_absmax
from ..kernels.fused import (
    causal_softmax_q,
    gelu_q,
    layer_norm_fwd_fused_single_pass_q,
    linear_a8_w8_bfp32_ofp32_GeLu_Q,
)
from .linear import _W8A8Base


class _LayerNormBuffers(torch.nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.input_scale = 1.0
        self.eps = eps
        self.register_buffer("weight", torch.ones(dim, dtype=torch.float32))
        self.register_buffer("bias", torch.zeros(dim, dtype=torch.float32))

    @classmethod
    def from_float(cls, module: torch.nn.LayerNorm, output_scale: float):
        """Folds the output scale into gamma and beta (reference nn/fused.py:49-57)."""
        n = module.normalized_shape[0]
        assert n == module.weight.numel() and n == module.bias.numel()
        q = cls(n, module.eps)
        q.weight = (module.weight / output_scale).detach()
        q.bias = (module.bias / output_scale).detach()
        return q


class _LayerNormQ(_LayerNormBuffers):
    """Pure-torch form: round half to even, then clamp (reference nn/fused.py:8-32)."""

    def forward(self, x):
        x = x.to(self.weight.dtype)
        y = torch.nn.functional.layer_norm(x, x.shape[-1:], self.weight, self.bias, self.eps)
        return y.round().clamp(-128, 127).to(torch.int8)


class LayerNormQ(_LayerNormBuffers):
    """LayerNorm -> int8 through the fused kernel (reference nn/fused.py:34-57)."""

    def forward(self, x):
        return layer_norm_fwd_fused_single_pass_q(x.to(self.weight.dtype), self.weight, self.bias, self.eps)


class DQ_Add_LayerNorm_Q(_LayerNormBuffers):
    """(residual_out_fp32, ln_out_int8) = f(residual_in_fp32, acc_int32): dequantise
    with ``input_scale``, add to the residual stream, LayerNorm, quantise
    (reference nn/fused.py:59-78; there the call ends in an undefined name).
    ``input_scale`` may be a float or a 0-dim tensor."""

    def forward(self, residual_input_fp, input_int32):
        return dq_add_layernorm_q_cpp(input_int32, self.input_scale, residual_input_fp,
                                      self.weight, self.bias, self.eps)


class GeLu_Q(torch.nn.Module):
    """Stand-alone quantising GELU: ``gelu_tanh(input_scale * x) * a`` cast back to
    x's dtype (reference nn/fused.py:81-87, whose forward calls a jit function from
    the host and cannot run).  int8 inputs take the CUDA kernel; ``input_scale``
    (default 1, the reference has none) de-quantises them first."""

    def __init__(self, alpha=1, input_scale=1.0):
        super().__init__()
        self.register_buffer("a", torch.tensor(alpha))
        self.input_scale = input_scale

    @torch.no_grad()
    def forward(self, x):
        if x.dtype == torch.int8:
            return gelu_q(x, self.input_scale, float(self.a))
        v = x.to(torch.float32) * self.input_scale
        y = 0.5 * v * (1 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v * v * v))) * self.a
        return y.to(x.dtype)


class CausalSoftmaxQ(torch.nn.Module):
    """int8(out_mul * softmax(causal_mask(scores))): the caller-side step between the
    two attention BMMs (not a reference class)."""

    def __init__(self, out_mul=127.0, causal=True):
        super().__init__()
        self.out_mul, self.causal = out_mul, causal

    @torch.no_grad()
    def forward(self, scores):
        return causal_softmax_q(scores, self.out_mul, self.causal)


class W8A8BFP32OFP32_GeLu_Q(_W8A8Base):
    """fc1 + GELU + quantise: int8 in, fp32 bias (not scaled), int8 out; ``b`` holds
    1/out_scale (reference nn/fused.py:90-151)."""

    BIAS_DTYPE = torch.float32

    def _op(self, x):
        return linear_a8_w8_bfp32_ofp32_GeLu_Q(x, self.weight, self.bias, self.a, self.b)

    @classmethod
    def from_float(cls, module: torch.nn.Linear, input_scale, out_scale):
        q = cls(module.in_features, module.out_features)
        q.weight, weight_scale = quantize_per_tensor_absmax(module.weight)
        q.bias = module.bias.to(torch.float32)
        q.a = input_scale * weight_scale
        q.input_scale, q.weight_scale = input_scale, weight_scale
        q.b = torch.tensor(1 / out_scale, dtype=q.b.dtype, device=q.b.device)
        return q
