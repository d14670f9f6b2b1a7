"""Shared launcher of the int8 GEMM / BMM entry point (ti_gemm_i8)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib, config

_SCALAR_CACHE = {}


def scale_tensor(s, device) -> torch.Tensor:
    """Return a 0-dim fp32 tensor on `device` holding `s`.

    The reference reads its scales on the device (tl.load(scale_a),
    kernels/linear.py:227,247), so a 0-dim CUDA tensor is the native form; Python
    numbers are accepted as a convenience and cached per (value, device)."""
    if torch.is_tensor(s):
        if s.numel() != 1:
            raise AssertionError("scale must hold exactly one element")
        if s.device != device or s.dtype != torch.float32:
            s = s.detach().to(device=device, dtype=torch.float32)
        return s.reshape(())
    key = (float(s), device)
    t = _SCALAR_CACHE.get(key)
    if t is None:
        t = torch.tensor(float(s), dtype=torch.float32, device=device)
        _SCALAR_CACHE[key] = t
    return t


def gemm(a3, b3, b_is_nk, out_dtype, epilogue, *, bias=None, alpha=None, beta=None, out=None,
         causal=False, rounding=None, path=None, residual=None):
    """a3: int8 [B,M,K] view (any strides).  b3: int8 [B,N,K] (b_is_nk) or [B,K,N].
    Returns the [B,M,N] result (written into `out` when given)."""
    _lib.require_cuda(a3, b3, bias, out)
    if a3.dtype != torch.int8 or b3.dtype != torch.int8:
        raise RuntimeError("int8 operands expected")
    lib = _lib.load()
    dev = a3.device
    B, M, K = a3.shape
    if b_is_nk:
        _, N, _ = b3.shape
        bsn, bsk = b3.stride(1), b3.stride(2)
    else:
        _, _, N = b3.shape
        bsn, bsk = b3.stride(2), b3.stride(1)
    if out is None:
        c = torch.empty((B, M, N), device=dev, dtype=out_dtype)
    else:
        if out.dtype != out_dtype or out.numel() != B * M * N or out.device != dev:
            raise AssertionError("out has the wrong dtype, size or device")
        c = out.view(B, M, N)
    p = _lib.GemmParams()
    p.a, p.b, p.c = a3.data_ptr(), b3.data_ptr(), c.data_ptr()
    keep = []
    if bias is not None:
        if bias.numel() != N:
            raise AssertionError("bias must have N elements")
        if not bias.is_contiguous():
            bias = bias.contiguous()
        keep.append(bias)
        p.bias = bias.data_ptr()
        p.bias_dtype = _lib.DTYPE_CODE[bias.dtype]
    if alpha is not None:
        alpha = scale_tensor(alpha, dev)
        keep.append(alpha)
        p.alpha = alpha.data_ptr()
    if beta is not None:
        beta = scale_tensor(beta, dev)
        keep.append(beta)
        p.beta = beta.data_ptr()
    p.m, p.n, p.k, p.batch = M, N, K, B
    p.a_stride_m, p.a_stride_k, p.a_stride_batch = a3.stride(1), a3.stride(2), a3.stride(0)
    p.b_stride_n, p.b_stride_k, p.b_stride_batch = bsn, bsk, b3.stride(0)
    p.c_stride_m, p.c_stride_n, p.c_stride_batch = c.stride(1), c.stride(2), c.stride(0)
    p.out_dtype = _lib.DTYPE_CODE[out_dtype]
    p.epilogue = epilogue
    p.rounding = config.rounding_mode() if rounding is None else rounding
    p.path = config.gemm_path() if path is None else path
    p.causal = 1 if causal else 0
    if residual is not None:
        # dequantise + residual-add epilogue: fp32 [M, N], columns contiguous
        _lib.require_cuda(residual)
        if residual.dtype != torch.float32 or residual.dim() != 2 or tuple(residual.shape) != (M, N) or B != 1:
            raise AssertionError("residual must be an fp32 [M, N] matrix (non-batched linear)")
        if residual.stride(1) != 1:
            residual = residual.contiguous()
        keep.append(residual)
        p.residual, p.residual_stride_m = residual.data_ptr(), residual.stride(0)
    with torch.cuda.device(dev):
        p.stream = _lib.current_stream_ptr(dev)
        if B == 1 and M <= 256:
            # few output tiles: let the library split K; the scratch comes from torch's allocator
            need = lib.ti_gemm_workspace_bytes(C.byref(p))
            if need > 0:
                ws = torch.empty(need, dtype=torch.uint8, device=dev)
                keep.append(ws)
                p.workspace, p.workspace_bytes = ws.data_ptr(), need
        rc = lib.ti_gemm_i8(C.byref(p))
    _lib.check(rc, "ti_gemm_i8")
    return c
