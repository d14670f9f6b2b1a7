"""CPU restatement of the reference's INT8 operator arithmetic.

TEST INFRASTRUCTURE ONLY: this module is the checker for the CUDA path (used by
``tests/``, the smoke check and the CPU-baseline leg of the benchmark).  Nothing
that ships may route through it.

Every function cites the reference lines it follows (paths are relative to the
reference project root).  The reference has no golden vectors of its own; the
restatement is pinned instead against outputs of the reference's own kernels
executed under Triton's CPU interpreter (``tests/golden/*.npz``, produced by
``tests/golden/make_golden.py``), and ``tests/test_oracle_golden.py`` holds the
comparison.

Conventions
-----------
* integer accumulation is exact: int8 x int8 products summed in int32.  It is
  evaluated here through float64 matmul, exact while K * 127^2 < 2^53.
* fp32 epilogues are evaluated operation by operation in IEEE fp32 without
  fused multiply-add, which is what the interpreter (numpy) does.
* two float->int8 casts exist:
    ``trunc_wrap``  truncate toward zero, keep the low byte.  This is what the
                    reference kernels' ``.to(tl.int8)`` does (kernels/linear.py:254).
    ``rne_sat``     round half to even, saturate to [-128, 127].
"""
from __future__ import annotations

import math

import numpy as np
import torch

SQRT_2_OVER_PI = math.sqrt(2.0 / math.pi)  # kernels/fused.py:13

TRUNC_WRAP = "trunc_wrap"
RNE_SAT = "rne_sat"


# --------------------------------------------------------------------------- casts
def cast_i8(f: torch.Tensor, mode: str) -> torch.Tensor:
    """float32 -> int8 under the named policy."""
    f = f.float()
    if mode == TRUNC_WRAP:
        # numpy astype(int8) on the interpreter == fptosi + low byte on the GPU
        return f.to(torch.int32).to(torch.int8)
    if mode == RNE_SAT:
        return f.round().clamp(-128, 127).to(torch.int8)
    raise ValueError(mode)


def _scalar(s) -> torch.Tensor:
    if torch.is_tensor(s):
        return s.detach().float().cpu().reshape(())
    return torch.tensor(float(s), dtype=torch.float32)


# --------------------------------------------------------------------------- accumulators
def acc_linear(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """int32 [M,N] = a[M,K] . w[N,K]^T   (K loop, kernels/linear.py:228-245)."""
    a2 = a.reshape(-1, a.shape[-1])
    assert a2.shape[1] == w.shape[1]
    if a2.shape[1] == 0:
        return torch.zeros(a2.shape[0], w.shape[0], dtype=torch.int32)
    out = a2.double() @ w.double().t()
    return out.to(torch.int64).to(torch.int32)


def acc_bmm_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """int32 [B,M,N] = a[B,M,K] . b[B,N,K]^T   (kernels/bmm.py:163-273)."""
    assert a.dim() == 3 and b.dim() == 3 and a.shape[0] == b.shape[0] and a.shape[2] == b.shape[2]
    return torch.bmm(a.double(), b.double().transpose(1, 2)).to(torch.int64).to(torch.int32)


def acc_bmm_nn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """int32 [B,M,N] = a[B,M,K] . b[B,K,N]   (kernels/bmm.py:12-122)."""
    assert a.dim() == 3 and b.dim() == 3 and a.shape[0] == b.shape[0] and a.shape[2] == b.shape[1]
    return torch.bmm(a.double(), b.double()).to(torch.int64).to(torch.int32)


def _lead(a, n):
    return tuple(a.shape[:-1]) + (n,)


# --------------------------------------------------------------------------- linears
def linear_a8_w8_ofp32(a, w, scale, dtype=torch.float32):
    """(scale * acc).to(dtype)   kernels/linear.py:107."""
    acc = acc_linear(a, w)
    return (_scalar(scale) * acc.float()).to(dtype).reshape(_lead(a, w.shape[0]))


def _scale_bias(acc, bias, alpha, beta):
    # c = 0 + f32(bias)*beta ; c += f32(acc)*alpha   kernels/linear.py:225-227,247
    c = bias.float()[None, :] * _scalar(beta)
    return c + acc.float() * _scalar(alpha)


def linear_a8_w8_b8_o8(a, w, bias, alpha, beta, mode=TRUNC_WRAP):
    """int8(beta*bias + alpha*acc)   kernels/linear.py:225-227,247,254."""
    f = _scale_bias(acc_linear(a, w), bias, alpha, beta)
    return cast_i8(f, mode).reshape(_lead(a, w.shape[0]))


def linear_a8_w8_b8_o8_f32(a, w, bias, alpha, beta):
    """The fp32 value the int8 cast of linear_a8_w8_b8_o8 is applied to."""
    return _scale_bias(acc_linear(a, w), bias, alpha, beta).reshape(_lead(a, w.shape[0]))


def linear_relu_a8_w8_b8_o8(a, w, bias, alpha, beta, mode=TRUNC_WRAP):
    """max(int8(...), 0): the cast comes first, then ReLU   kernels/linear.py:396."""
    y = linear_a8_w8_b8_o8(a, w, bias, alpha, beta, mode)
    return torch.clamp_min(y, 0)


def linear_a8_w8_b32_o32(a, w, bias):
    """acc + bias in wrapping int32   kernels/linear.py:505-507,534."""
    acc = acc_linear(a, w).to(torch.int64) + bias.to(torch.int64)[None, :]
    acc = ((acc + 2**31) % 2**32) - 2**31
    return acc.to(torch.int32).reshape(_lead(a, w.shape[0]))


def linear_a8_w8_b32_o32_with_scaling(a, w, bias, alpha, beta):
    """int32(trunc(beta*f32(bias) + alpha*f32(acc)))   kernels/linear.py:646,666,674."""
    f = _scale_bias(acc_linear(a, w), bias, alpha, beta)
    return f.to(torch.int32).reshape(_lead(a, w.shape[0]))


def linear_a8_w8_bfp32_ofp32(a, w, bias, alpha, beta, dtype=None):
    """beta*f32(bias) + alpha*f32(acc), stored in the bias dtype by default
    kernels/linear.py:788,809,817,829-832."""
    if dtype is None:
        dtype = bias.dtype
    f = _scale_bias(acc_linear(a, w), bias, alpha, beta)
    return f.to(dtype).reshape(_lead(a, w.shape[0]))


def gelu_tanh_scaled(v: torch.Tensor, scale) -> torch.Tensor:
    """0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x*x*x)))*scale, left to right in fp32
    kernels/fused.py:76-79."""
    v = v.float()
    c = torch.tensor(SQRT_2_OVER_PI, dtype=torch.float32)
    k = torch.tensor(0.044715, dtype=torch.float32)
    inner = c * (v + k * v * v * v)
    t = torch.from_numpy(np.tanh(inner.numpy()))
    return torch.tensor(0.5, dtype=torch.float32) * v * (1 + t) * _scalar(scale)


def linear_a8_w8_bfp32_ofp32_gelu_q_f32(a, w, bias, alpha, scale_b):
    acc = acc_linear(a, w)
    v = acc.float() * _scalar(alpha) + bias.float()[None, :]  # bias is NOT scaled, kernels/fused.py:184-186
    return gelu_tanh_scaled(v, scale_b).reshape(_lead(a, w.shape[0]))


def linear_a8_w8_bfp32_ofp32_GeLu_Q(a, w, bias, alpha, scale_b, mode=TRUNC_WRAP):
    """int8(gelu(alpha*acc + bias) * scale_b)   kernels/fused.py:184-187."""
    return cast_i8(linear_a8_w8_bfp32_ofp32_gelu_q_f32(a, w, bias, alpha, scale_b), mode)


# --------------------------------------------------------------------------- BMMs
def bmm_s8t_s8n_s32t(a, b):
    return acc_bmm_nt(a, b)


def bmm_s8t_s8t_s32t(a, b):
    return acc_bmm_nn(a, b)


def bmm_s8t_s8n_f32t(a, b, scale, dtype=torch.float32):
    """f32(acc)*scale -> dtype   kernels/bmm.py:414,426."""
    return (acc_bmm_nt(a, b).float() * _scalar(scale)).to(dtype)


def bmm_s8t_s8n_s8t(a, b, scale, mode=TRUNC_WRAP):
    """int8(f32(acc)*scale)   kernels/bmm.py:562."""
    return cast_i8(acc_bmm_nt(a, b).float() * _scalar(scale), mode)


def bmm_s8t_s8t_s8t(a, b, scale, mode=TRUNC_WRAP):
    """NN-layout variant   kernels/bmm.py:710."""
    return cast_i8(acc_bmm_nn(a, b).float() * _scalar(scale), mode)


# --------------------------------------------------------------------------- LayerNorm family
def _ln_block_size(n: int, elem_size: int) -> int:
    # kernels/fused.py:359-362
    max_fused = 65536 // elem_size
    p2 = 1 << max(0, (n - 1).bit_length())
    return min(max(min(max_fused, p2), 128), 4096)


def layer_norm_stats(x32: np.ndarray, block: int, rms: bool):
    """Row mean and variance with the reference's blocked update
    (kernels/fused.py:276-308), vectorised over rows.  x32: float32 [rows, N]."""
    rows, n = x32.shape
    mean = np.zeros(rows, dtype=np.float32)
    var = np.zeros(rows, dtype=np.float32)
    for start in range(0, n, block):
        end = min(start + block, n)
        cnt = np.float32(end - start)
        a = np.zeros((rows, block), dtype=np.float32)
        a[:, : end - start] = x32[:, start:end]
        msk = np.zeros(block, dtype=np.float32)
        msk[: end - start] = 1.0
        if rms:
            var = var + np.sum(a * a, axis=1, dtype=np.float32)
        else:
            block_mean = np.sum(a, axis=1, dtype=np.float32) / cnt
            delta = block_mean - mean
            delta_sqr = delta * delta
            block_delta = np.sum((a - block_mean[:, None]) * a, axis=1, dtype=np.float32)
            mean = mean + np.sum((a - mean[:, None]) * msk[None, :], axis=1, dtype=np.float32) / np.float32(end)
            var = var + (block_delta + delta_sqr * np.float32(start * (end - start)) / np.float32(end))
    var = var / np.float32(n)
    return mean, var


def layer_norm_f32(x, weight, bias, eps, use_rms_norm=False):
    """fp32 value before the output cast of the reference LayerNorm kernels
    (kernels/fused.py:271-331): ((a-mean)*rstd)*w (+b)."""
    n = x.shape[-1]
    elem = x.element_size()
    if x.dtype == torch.float16:
        eps = max(eps, 1.6e-5)  # kernels/fused.py:352-353
    x32 = x.reshape(-1, n).float().numpy()
    block = _ln_block_size(n, elem)
    mean, var = layer_norm_stats(x32, block, use_rms_norm)
    rstd = np.float32(1.0) / np.sqrt(var + np.float32(eps))
    out = (x32 - mean[:, None]) * rstd[:, None]
    out = out * weight.float().numpy()[None, :]
    if bias is not None:
        out = out + bias.float().numpy()[None, :]
    return torch.from_numpy(out.astype(np.float32)).reshape(x.shape)


def layer_norm_fwd_fused_single_pass_q(x, weight, bias, eps, use_rms_norm=False, mode=TRUNC_WRAP):
    """kernels/fused.py:235-382: LayerNorm then int8 cast (:331)."""
    return cast_i8(layer_norm_f32(x, weight, bias, eps, use_rms_norm), mode)


def layer_norm_fwd_fused_single_pass(x, weight, bias, eps, use_rms_norm=False):
    """kernels/fused.py:385-532: LayerNorm stored in the input dtype."""
    return layer_norm_f32(x, weight, bias, eps, use_rms_norm).to(x.dtype)


def skip_layer_norm_fwd_fused_single_pass2(x, skip, weight, bias, eps, use_rms_norm=False):
    """kernels/fused.py:696-862: (LN(x), LN(x).to(dtype) + skip)."""
    out = layer_norm_f32(x, weight, bias, eps, use_rms_norm).to(x.dtype)
    return out, (out + skip.reshape(x.shape)).to(x.dtype)


def skip_layer_norm_fwd_fused_single_pass(x, skip, weight, bias, eps, use_rms_norm=False):
    """kernels/fused.py:535-693: LN(x).to(dtype) + skip."""
    return skip_layer_norm_fwd_fused_single_pass2(x, skip, weight, bias, eps, use_rms_norm)[1]


def dq_add_layernorm_q(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """functional/fused.py:6-15, the only executable definition of the fused
    dequant -> residual add -> LayerNorm -> quant op: clamp first, then round half
    to even."""
    residual_output_fp = torch.add(residual_input_fp, input_int32, alpha=float(input_scale_fp))
    ln = torch.nn.functional.layer_norm(
        residual_output_fp, residual_output_fp.shape[-1:], gamma, beta, eps)
    return residual_output_fp, ln.clamp(-128, 127).round().to(torch.int8)


def dq_add_layernorm_q_f32(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """fp32 LayerNorm value of dq_add_layernorm_q before the clamp/round."""
    r = torch.add(residual_input_fp, input_int32, alpha=float(input_scale_fp))
    return r, torch.nn.functional.layer_norm(r, r.shape[-1:], gamma, beta, eps)


# --------------------------------------------------------------------------- element-wise / row ops around the path
def gelu_q(x_i8, in_scale, out_mul, mode=RNE_SAT):
    """Stand-alone int8 GELU: int8(gelu_tanh(in_scale * x) * out_mul), the formula
    of fast_geluQ (kernels/fused.py:76-79) on a dequantised int8 input.  The
    reference module that was meant to expose it (nn/fused.py:81-87) calls a jit
    function from the host and cannot run, so no reference output exists for it."""
    v = x_i8.float() * _scalar(in_scale)
    return cast_i8(gelu_tanh_scaled(v, out_mul), mode)


def causal_softmax_q(s_f32, out_mul=127.0, mode=RNE_SAT):
    """int8(out_mul * softmax(mask_causal(s), dim=-1)) for s [B,M,N] with query row
    i attending keys j <= i + (N - M).  Not part of the reference (it leaves the
    softmax between its two attention BMMs to the caller); defined by the
    attention configuration of the benchmark plan."""
    b, m, n = s_f32.shape
    i = torch.arange(m)[:, None]
    j = torch.arange(n)[None, :]
    masked = s_f32.float().masked_fill(j > i + (n - m), float("-inf"))
    p = torch.softmax(masked, dim=-1)
    return cast_i8(p * _scalar(out_mul), mode)
