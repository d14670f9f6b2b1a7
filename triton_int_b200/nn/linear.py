"""W8A8 linear modules: the class names, buffers (``weight``, ``bias``, ``a``,
``b``), constructors and ``from_float`` signatures of the reference's
``triton_int/nn/linear.py``, so a ``state_dict`` moves between the two unchanged.
"""
from __future__ import annotations

import torch

from ..functional.quantization import (
    fake_quantize_activation_per_tensor_absmax,
    fake_quantize_activation_per_token_absmax,
    quantize_per_tensor_absmax,
    quantize_weight_per_channel_absmax,
)
from ..kernels.linear import (
    linear_a8_w8_b8_o8,
    linear_a8_w8_b32_o32,
    linear_a8_w8_b32_o32_with_scaling,
    linear_a8_w8_bfp32_ofp32,
    linear_relu_a8_w8_b8_o8,
)


class _W8A8Base(torch.nn.Module):
    """int8 weight [out, in] plus a bias of the subclass's dtype and two 0-dim scales."""

    BIAS_DTYPE = torch.int8
    DEFAULT_BETA = None  # None: take the constructor argument

    def __init__(self, in_features, out_features, alpha=1.0, beta=1.0):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("weight", torch.randint(-127, 127, (out_features, in_features), dtype=torch.int8))
        self.register_buffer("bias", torch.zeros(out_features, dtype=self.BIAS_DTYPE))
        self.register_buffer("a", torch.tensor(alpha))
        self.register_buffer("b", torch.tensor(beta if self.DEFAULT_BETA is None else self.DEFAULT_BETA))

    def _op(self, x2d):
        raise NotImplementedError

    @torch.no_grad()
    def forward(self, x):
        lead = x.shape[:-1]
        y = self._op(x.reshape(-1, x.shape[-1]))
        return y.view(*lead, -1)


class W8A8B8O8Linear(_W8A8Base):
    """q/k/v projections: int8 in, int8 bias, int8 out (reference nn/linear.py:18-67)."""

    def _op(self, x):
        return linear_a8_w8_b8_o8(x, self.weight, self.bias, self.a, self.b)

    @classmethod
    def from_float(cls, module: torch.nn.Linear, input_scale, output_scale):
        q = cls(module.in_features, module.out_features)
        q.weight, weight_scale = quantize_per_tensor_absmax(module.weight)
        q.bias, bias_scale = quantize_per_tensor_absmax(module.bias)
        q.a = input_scale * weight_scale / output_scale
        q.b = bias_scale / output_scale
        return q


class W8A8B8O8LinearReLU(W8A8B8O8Linear):
    """fc1 with ReLU applied to the int8 result (reference nn/linear.py:70-122)."""

    def _op(self, x):
        return linear_relu_a8_w8_b8_o8(x, self.weight, self.bias, self.a, self.b)


class W8A8B32O32LinearWithoutScaling(_W8A8Base):
    """Raw int32 accumulators plus an int32 bias (reference nn/linear.py:125-159)."""

    BIAS_DTYPE = torch.int32

    def __init__(self, in_features, out_features):
        super().__init__(in_features, out_features)
        del self._buffers["a"], self._buffers["b"]

    def _op(self, x):
        return linear_a8_w8_b32_o32(x, self.weight, self.bias)


class W8A8B32O32Linear(_W8A8Base):
    """fc2 / out_proj with int32 bias and int32 output (reference nn/linear.py:162-219)."""

    BIAS_DTYPE = torch.int32

    def _op(self, x):
        return linear_a8_w8_b32_o32_with_scaling(x, self.weight, self.bias, self.a, self.b)

    @classmethod
    def from_float(cls, module: torch.nn.Linear, input_scale, output_scale):
        q = cls(module.in_features, module.out_features)
        q.weight, weight_scale = quantize_per_tensor_absmax(module.weight)
        module.bias = torch.nn.Parameter(module.bias.float(), requires_grad=False)
        bias_scale = module.bias.abs().max() / (2**31 - 1)
        q.bias = (module.bias / bias_scale).round().to(torch.int32)
        q.a = input_scale * weight_scale / output_scale
        q.b = bias_scale / output_scale
        q.input_scale, q.output_scale = input_scale, output_scale
        q.weight_scale, q.bias_scale = weight_scale, bias_scale
        return q


class W8A8BFP32OFP32Linear(_W8A8Base):
    """fc2 / out_proj with a floating bias; the output takes the bias dtype
    (reference nn/linear.py:222-278).  ``b`` is fixed at 1."""

    BIAS_DTYPE = torch.float32
    DEFAULT_BETA = 1.0

    def _op(self, x):
        return linear_a8_w8_bfp32_ofp32(x, self.weight, self.bias, self.a, self.b)

    @classmethod
    def from_float(cls, module: torch.nn.Linear, input_scale):
        q = cls(module.in_features, module.out_features)
        q.weight, weight_scale = quantize_per_tensor_absmax(module.weight)
        q.bias = module.bias.to(torch.float32)
        q.a = input_scale * weight_scale
        q.input_scale, q.weight_scale = input_scale, weight_scale
        return q


class DynamicW8A8BFP32OFP32Linear(_W8A8Base):
    """Per-tensor dynamic activation quantisation in front of the fp32-output
    linear.  The reference class of this purpose (nn/linear.py:281-342,
    ``DanymicW8A8BFP32OFP32Linear``) cannot be constructed (it registers one
    buffer twice); this is the working form, also exported under that name."""

    BIAS_DTYPE = torch.float32
    DEFAULT_BETA = 1.0

    def __init__(self, in_features, out_features, alpha=1.0, beta=1.0):
        super().__init__(in_features, out_features, alpha, beta)
        self.register_buffer("weight_scale", torch.tensor(alpha))

    def _op(self, x):
        from ..functional.quantization import quantize_per_tensor_absmax_cuda
        xq, scale = quantize_per_tensor_absmax_cuda(x)   # fused absmax + quantise, x left untouched
        return linear_a8_w8_bfp32_ofp32(xq, self.weight, self.bias, scale.float() * self.weight_scale, self.b)

    @classmethod
    def from_float(cls, module: torch.nn.Linear):
        q = cls(module.in_features, module.out_features)
        q.weight, q.weight_scale = quantize_per_tensor_absmax(module.weight)
        q.bias = module.bias.to(torch.float32)
        return q


DanymicW8A8BFP32OFP32Linear = DynamicW8A8BFP32OFP32Linear


class W8A16Linear(torch.nn.Module):
    """int8 weight de-quantised to fp16 at run time, then a plain fp16 linear
    (reference nn/linear.py:345-417): no custom kernel is involved."""

    def __init__(self, in_features, out_features, bias=True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight", torch.randint(-127, 127, (out_features, in_features), dtype=torch.int8))
        self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16) if bias else None)
        self.register_buffer("weight_scales", torch.ones(out_features, dtype=torch.float16))

    def _dequantised_weight(self):
        scales = self.weight_scales
        if scales.numel() == self.out_features:
            scales = scales.view(-1, 1)
        return self.weight.to(torch.float16) * scales.to(torch.float16)

    @torch.no_grad()
    def forward(self, x):
        return torch.nn.functional.linear(x, self._dequantised_weight(), self.bias)

    @classmethod
    def from_float(cls, module, weight_quant="per_channel"):
        assert isinstance(module, torch.nn.Linear)
        q = cls(module.in_features, module.out_features, module.bias is not None)
        if weight_quant == "per_channel":
            q.weight, q.weight_scales = quantize_weight_per_channel_absmax(module.weight)
        elif weight_quant == "per_tensor":
            q.weight, q.weight_scales = quantize_per_tensor_absmax(module.weight)
        else:
            raise ValueError('weight_quant must be "per_channel" or "per_tensor"')
        if module.bias is not None:
            q.bias = module.bias.to(torch.float16)
        return q

    def extra_repr(self):
        return f"{self.in_features}, {self.out_features}, bias={self.bias is not None}"


class W8FakeA8Linear(W8A16Linear):
    """W8A16Linear behind a fake-quantised activation (reference nn/linear.py:420-491)."""

    def __init__(self, in_features, out_features, bias=True, act_quant="per_token"):
        super().__init__(in_features, out_features, bias)
        if act_quant == "per_token":
            self.activation_fake_quantizer = fake_quantize_activation_per_token_absmax
        elif act_quant == "per_tensor":
            self.activation_fake_quantizer = fake_quantize_activation_per_tensor_absmax
        else:
            raise ValueError('act_quant must be "per_token" or "per_tensor"')

    @torch.no_grad()
    def forward(self, x):
        return super().forward(self.activation_fake_quantizer(x))

    @classmethod
    def from_float(cls, module, act_quant="per_token"):
        assert isinstance(module, torch.nn.Linear)
        q = cls(module.in_features, module.out_features, module.bias is not None, act_quant)
        q.weight, q.weight_scales = quantize_weight_per_channel_absmax(module.weight)
        if module.bias is not None:
            q.bias = module.bias.to(torch.float16)
        return q
