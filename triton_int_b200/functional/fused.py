"""Dequant -> residual add -> LayerNorm (-> quant), functional form
(reference functional/fused.py:6-32)."""
import torch

from ..kernels.fused import dq_add_layernorm_q


def dq_add_layernorm_q_py(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """The torch definition (reference functional/fused.py:6-15): separate torch ops,
    clamp to [-128,127] then round half to even.  Kept for comparison; the modules
    call dq_add_layernorm_q_cpp."""
    residual_output_fp = torch.add(residual_input_fp, input_int32, alpha=input_scale_fp)
    ln_output_fp = torch.nn.functional.layer_norm(
        residual_output_fp, residual_output_fp.shape[-1:], gamma, beta, eps)
    return residual_output_fp, ln_output_fp.clamp(-128, 127).round().to(torch.int8)


def dq_add_layernorm(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """Same without the final quantisation (reference functional/fused.py:18-24)."""
    residual_output_fp = torch.add(residual_input_fp, input_int32, alpha=input_scale_fp)
    ln_output_fp = torch.nn.functional.layer_norm(
        residual_output_fp, residual_output_fp.shape[-1:], gamma, beta, eps)
    return residual_output_fp, ln_output_fp


def dq_add_layernorm_q_cpp(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """The fused CUDA kernel (one pass over each row).  In the reference this name
    forwards to an operator that is never imported (functional/fused.py:3,27-32)."""
    return dq_add_layernorm_q(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps)
