"""Fused / memory-bound operators: the GELU-quantising linear, the LayerNorm
family, and the three row operators the reference leaves undefined or to the
caller (dequant+add+LayerNorm+quant, stand-alone int8 GELU, causal softmax->int8).
Names and signatures of the first two groups follow the reference's
``triton_int/kernels/fused.py``.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib, config
from . import register_torch_op
from ._gemm import gemm, scale_tensor


@register_torch_op("(Tensor a, Tensor b, Tensor bias, Tensor scale_a, Tensor scale_b, Tensor? out=None) -> Tensor")
def linear_a8_w8_bfp32_ofp32_GeLu_Q(a, b, bias, scale_a, scale_b, out=None):
    """int8(gelu_tanh(scale_a * acc + bias) * scale_b); the bias is NOT scaled
    -- reference kernels/fused.py:88-231 (epilogue :184-187)."""
    assert b.dim() == 2
    assert a.shape[-1] == b.shape[1], "Incompatible dimensions"
    lead = a.shape[:-1]
    a3 = a.reshape(-1, a.shape[-1]).unsqueeze(0)
    c = gemm(a3, b.unsqueeze(0), True, torch.int8, _lib.EPI_GELU_Q, bias=bias, alpha=scale_a, beta=scale_b, out=out)
    return c.view(*lead, b.shape[0])


def _layernorm(x, weight, bias, eps, use_rms_norm, out_dtype, *, skip=None, want_out=True, want_out2=False,
               int32_in=None, residual=None, dq_scale=1.0, bias_i32=None, want_residual_out=False):
    src = x if int32_in is None else int32_in
    _lib.require_cuda(src, weight, bias, skip, residual, bias_i32)
    lib = _lib.load()
    n = src.shape[-1]
    dev = src.device
    assert weight.numel() == n
    if int32_in is None:
        assert x.dtype == weight.dtype, f"input and weight bias must have the same dtype: {x.dtype}, {weight.dtype}"
        if bias is not None:
            assert x.dtype == bias.dtype, f"input and bias must have the same dtype: {x.dtype}, {bias.dtype}"
        if x.dtype == torch.float16:
            eps = max(eps, 1.6e-5)  # reference kernels/fused.py:352-353
    x2 = src.reshape(-1, n)
    rows = x2.shape[0]
    s2 = None
    if want_out2:
        s2 = skip.reshape(-1, n)
        assert s2.shape == x2.shape
        if s2.stride() != x2.stride():  # the kernel walks skip with x's strides (reference kernels/fused.py:625-630)
            x2, s2 = x2.contiguous(), s2.contiguous()
    p = _lib.LayerNormParams()
    keep = [x2, s2]
    p.x = x2.data_ptr()
    p.x_dtype = _lib.DTYPE_CODE[x2.dtype]
    p.param_dtype = _lib.DTYPE_CODE[weight.dtype]
    p.out_dtype = _lib.DTYPE_CODE[out_dtype]
    w = weight if weight.is_contiguous() else weight.contiguous()
    p.gamma = w.data_ptr()
    keep.append(w)
    if bias is not None:
        bb = bias if bias.is_contiguous() else bias.contiguous()
        p.beta = bb.data_ptr()
        keep.append(bb)
    p.rows, p.n = rows, n
    p.x_row_stride, p.x_col_stride = x2.stride(0) if rows > 1 else n, x2.stride(1)
    out = out2 = res_out = None
    if want_out:
        out = torch.empty(src.shape, device=dev, dtype=out_dtype)
        p.out = out.data_ptr()
    if want_out2:
        out2 = torch.empty(src.shape, device=dev, dtype=out_dtype)
        p.out2 = out2.data_ptr()
        p.skip = s2.data_ptr()
    p.out_row_stride, p.out_col_stride = n, 1
    if int32_in is not None:
        r2 = residual.reshape(-1, n)
        if r2.dtype != torch.float32 or not r2.is_contiguous():
            r2 = r2.float().contiguous()
        keep.append(r2)
        p.residual_in = r2.data_ptr()
        if want_residual_out:
            res_out = torch.empty(src.shape, device=dev, dtype=torch.float32)
            p.residual_out = res_out.data_ptr()
        if bias_i32 is not None:
            bi = bias_i32.contiguous()
            keep.append(bi)
            p.bias_i32 = bi.data_ptr()
        if torch.is_tensor(dq_scale):
            ds = scale_tensor(dq_scale, dev)
            keep.append(ds)
            p.dq_scale_dev = ds.data_ptr()
        else:
            p.dq_scale = float(dq_scale)
    p.eps = float(eps)
    p.rounding = config.rounding_mode()
    p.rms = 1 if use_rms_norm else 0
    with torch.cuda.device(dev):
        p.stream = _lib.current_stream_ptr(dev)
        rc = lib.ti_layernorm(C.byref(p))
    _lib.check(rc, "ti_layernorm")
    return out, out2, res_out


@register_torch_op("(Tensor x, Tensor weight, Tensor? bias, float eps, bool use_rms_norm=False) -> Tensor")
def layer_norm_fwd_fused_single_pass_q(x, weight, bias, eps, use_rms_norm=False):
    """int8(LayerNorm(x) * weight + bias)   -- reference kernels/fused.py:235-382."""
    return _layernorm(x, weight, bias, eps, use_rms_norm, torch.int8)[0]


@register_torch_op("(Tensor x, Tensor weight, Tensor? bias, float eps, bool use_rms_norm=False) -> Tensor")
def layer_norm_fwd_fused_single_pass(x, weight, bias, eps, use_rms_norm=False):
    """LayerNorm in the input dtype   -- reference kernels/fused.py:385-532."""
    return _layernorm(x, weight, bias, eps, use_rms_norm, x.dtype)[0]


@register_torch_op("(Tensor x, Tensor skip, Tensor weight, Tensor? bias, float eps, bool use_rms_norm=False) -> Tensor")
def skip_layer_norm_fwd_fused_single_pass(x, skip, weight, bias, eps, use_rms_norm=False):
    """LayerNorm(x) + skip   -- reference kernels/fused.py:535-693."""
    return _layernorm(x, weight, bias, eps, use_rms_norm, x.dtype, skip=skip, want_out=False, want_out2=True)[1]


@register_torch_op("(Tensor x, Tensor skip, Tensor weight, Tensor? bias, float eps, bool use_rms_norm=False) -> (Tensor, Tensor)")
def skip_layer_norm_fwd_fused_single_pass2(x, skip, weight, bias, eps, use_rms_norm=False):
    """(LayerNorm(x), LayerNorm(x) + skip)   -- reference kernels/fused.py:696-862."""
    o, o2, _ = _layernorm(x, weight, bias, eps, use_rms_norm, x.dtype, skip=skip, want_out=True, want_out2=True)
    return o, o2


@register_torch_op("(Tensor input_int32, Tensor input_scale_fp, Tensor residual_input_fp, Tensor gamma, Tensor? beta, float eps, Tensor? bias_int32=None) -> (Tensor, Tensor)")
def dq_add_layernorm_q(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps, bias_int32=None):
    """(residual + scale * int32, int8(LayerNorm(that))) in one pass over the row.
    The operator the reference names but never defines (functional/fused.py:3,27-32;
    dead stub kernels/fused.py:17-61); semantics from functional/fused.py:6-15.
    ``input_scale_fp`` may be a Python float or a 0-dim tensor; ``bias_int32`` (an
    extension) is added to the int32 row before dequantisation."""
    assert input_int32.dtype == torch.int32
    out, _, res = _layernorm(None, gamma, beta, eps, False, torch.int8, int32_in=input_int32,
                             residual=residual_input_fp, dq_scale=input_scale_fp, bias_i32=bias_int32,
                             want_residual_out=True)
    return res, out


def gelu_q(x, in_scale, out_mul, out=None):
    """int8(gelu_tanh(in_scale * x_int8) * out_mul): the stand-alone int8 GELU
    (formula of fast_geluQ, reference kernels/fused.py:76-79)."""
    _lib.require_cuda(x, out)
    assert x.dtype == torch.int8
    xc = x if x.is_contiguous() else x.contiguous()
    y = torch.empty_like(xc) if out is None else out
    assert y.is_contiguous() and y.dtype == torch.int8 and y.numel() == xc.numel()
    with torch.cuda.device(x.device):
        rc = _lib.load().ti_gelu_q(xc.data_ptr(), y.data_ptr(), xc.numel(), float(in_scale), float(out_mul),
                                   config.rounding_mode(), _lib.current_stream_ptr(x.device))
    _lib.check(rc, "ti_gelu_q")
    return y


def causal_softmax_q(s, out_mul=127.0, causal=True, out=None):
    """int8(out_mul * softmax(mask(s), dim=-1)) for fp32 scores [B, M, N]; the step
    between bmm_s8t_s8n_f32t and bmm_s8t_s8n_s8t that the reference leaves to
    the caller."""
    _lib.require_cuda(s, out)
    assert s.dim() == 3 and s.dtype == torch.float32
    if s.stride(2) != 1:
        s = s.contiguous()
    B, M, N = s.shape
    p = torch.empty((B, M, N), device=s.device, dtype=torch.int8) if out is None else out
    assert p.shape == s.shape and p.dtype == torch.int8 and p.stride(2) == 1
    with torch.cuda.device(s.device):
        rc = _lib.load().ti_softmax_q(s.data_ptr(), p.data_ptr(), B, M, N, s.stride(1), s.stride(0),
                                      p.stride(1), p.stride(0), 1 if causal else 0, float(out_mul),
                                      config.rounding_mode(), _lib.current_stream_ptr(s.device))
    _lib.check(rc, "ti_softmax_q")
    return p


def attention_i8(q, k, v, alpha_qk, alpha_pv, p_mul=127.0, causal=True, out=None):
    """Fused int8 attention: int8(alpha_pv * P @ V) with P = int8(p_mul * softmax(mask(alpha_qk * Q @ K^T))).

    q [B, Sq, h, 128], k and v [B, Sk, h, 128] int8 views with arbitrary batch / row /
    head strides (for example slices of one [T, 3*H] projection buffer viewed as
    [B, S, h, D]); returns o [B, Sq, h, 128] int8.  Equivalent to
    bmm_s8t_s8n_f32t -> causal_softmax_q -> bmm_s8t_s8n_s8t on [B*h, S, D] operands
    (int8 P may differ by one step at rounding boundaries because the row sum is
    accumulated in a different order)."""
    _lib.require_cuda(q, k, v, out)
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4
    assert q.dtype == torch.int8 and k.dtype == torch.int8 and v.dtype == torch.int8
    B, Sq, H, D = q.shape
    assert k.shape == v.shape and k.shape[0] == B and k.shape[2] == H and k.shape[3] == D
    Sk = k.shape[1]
    for t in (q, k, v):
        assert t.stride(3) == 1, "the head dimension must be contiguous"
    o = torch.empty((B, Sq, H, D), device=q.device, dtype=torch.int8) if out is None else out
    assert o.shape == (B, Sq, H, D) and o.dtype == torch.int8 and o.stride(3) == 1
    dev = q.device
    a1, a2 = scale_tensor(alpha_qk, dev), scale_tensor(alpha_pv, dev)
    p = _lib.AttentionParams()
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.alpha_qk, p.alpha_pv = a1.data_ptr(), a2.data_ptr()
    p.batch, p.heads, p.seq_q, p.seq_k, p.head_dim = B, H, Sq, Sk, D
    p.q_stride_b, p.q_stride_s, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    p.k_stride_b, p.k_stride_s, p.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    p.v_stride_b, p.v_stride_s, p.v_stride_h = v.stride(0), v.stride(1), v.stride(2)
    p.o_stride_b, p.o_stride_s, p.o_stride_h = o.stride(0), o.stride(1), o.stride(2)
    p.p_mul = float(p_mul)
    p.causal = 1 if causal else 0
    p.rounding = config.rounding_mode()
    with torch.cuda.device(dev):
        p.stream = _lib.current_stream_ptr(dev)
        rc = _lib.load().ti_attention_i8(C.byref(p))
    _lib.check(rc, "ti_attention_i8")
    return o
