"""ctypes binding of the C ABI declared in include/triton_int_b200.h.

The product path has no CPU fallback: if the CUDA library is missing and cannot
be built, importing an operator raises; if a tensor is not on a CUDA device the
call raises.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _build

# ---- enums (mirror include/triton_int_b200.h) ----
TI_OK, TI_ERR_SHAPE, TI_ERR_DTYPE, TI_ERR_ALIGN, TI_ERR_DEVICE, TI_ERR_TIMEOUT, TI_ERR_CUDA, TI_ERR_UNSUPPORTED = range(8)
TI_I8, TI_I32, TI_F32, TI_F16, TI_BF16 = range(5)
ROUND_RNE_SAT, ROUND_TRUNC_WRAP = 0, 1
EPI_I32, EPI_SCALE, EPI_SCALE_BIAS, EPI_SCALE_BIAS_RELU, EPI_GELU_Q, EPI_DQ_ADD = range(6)
PATH_AUTO, PATH_TCGEN05, PATH_GENERIC = range(3)

DTYPE_CODE = {torch.int8: TI_I8, torch.int32: TI_I32, torch.float32: TI_F32,
              torch.float16: TI_F16, torch.bfloat16: TI_BF16}

EXPORTS = ["ti_gemm_i8", "ti_gemm_workspace_bytes", "ti_gemm_i8_static_scratch", "ti_static_scratch_bytes", "ti_layernorm", "ti_gelu_q", "ti_softmax_q", "ti_attention_i8", "ti_tp_reduce_layernorm_q", "ti_gemm_i8_scatter", "ti_tp_barrier", "ti_debug_expire_wait", "ti_quantize_absmax", "ti_device_status",
           "ti_version", "ti_last_error_string", "ti_launch_count", "ti_device_supported"]


class GemmParams(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("bias", C.c_void_p),
        ("alpha", C.c_void_p), ("beta", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("batch", C.c_int64),
        ("a_stride_m", C.c_int64), ("a_stride_k", C.c_int64), ("a_stride_batch", C.c_int64),
        ("b_stride_n", C.c_int64), ("b_stride_k", C.c_int64), ("b_stride_batch", C.c_int64),
        ("c_stride_m", C.c_int64), ("c_stride_n", C.c_int64), ("c_stride_batch", C.c_int64),
        ("bias_dtype", C.c_int32), ("out_dtype", C.c_int32), ("epilogue", C.c_int32),
        ("rounding", C.c_int32), ("path", C.c_int32), ("causal", C.c_int32),
        ("stream", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("residual", C.c_void_p), ("residual_stride_m", C.c_int64),
    ]


class LayerNormParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("residual_in", C.c_void_p), ("residual_out", C.c_void_p),
        ("bias_i32", C.c_void_p), ("gamma", C.c_void_p), ("beta", C.c_void_p), ("skip", C.c_void_p),
        ("out", C.c_void_p), ("out2", C.c_void_p), ("dq_scale_dev", C.c_void_p),
        ("rows", C.c_int64), ("n", C.c_int64),
        ("x_row_stride", C.c_int64), ("x_col_stride", C.c_int64),
        ("out_row_stride", C.c_int64), ("out_col_stride", C.c_int64),
        ("eps", C.c_float), ("dq_scale", C.c_float),
        ("x_dtype", C.c_int32), ("param_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("rounding", C.c_int32), ("rms", C.c_int32),
        ("stream", C.c_void_p),
    ]


class AttentionParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("alpha_qk", C.c_void_p), ("alpha_pv", C.c_void_p),
        ("batch", C.c_int64), ("heads", C.c_int64), ("seq_q", C.c_int64), ("seq_k", C.c_int64), ("head_dim", C.c_int64),
        ("q_stride_b", C.c_int64), ("q_stride_s", C.c_int64), ("q_stride_h", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_s", C.c_int64), ("k_stride_h", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_s", C.c_int64), ("v_stride_h", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_s", C.c_int64), ("o_stride_h", C.c_int64),
        ("p_mul", C.c_float), ("causal", C.c_int32), ("rounding", C.c_int32),
        ("stream", C.c_void_p),
    ]


class QuantizeParams(C.Structure):
    _fields_ = [("x", C.c_void_p), ("q", C.c_void_p), ("scales", C.c_void_p),
                ("rows", C.c_int64), ("n", C.c_int64), ("x_row_stride", C.c_int64), ("q_row_stride", C.c_int64),
                ("x_dtype", C.c_int32), ("per_token", C.c_int32), ("clamp_min", C.c_int32), ("stream", C.c_void_p)]


class GemmScatter(C.Structure):
    _fields_ = [("recv", C.c_void_p * 8), ("world", C.c_int32), ("rank", C.c_int32), ("rows_per_rank", C.c_int64)]


class TpReduceLnParams(C.Structure):
    _fields_ = [
        ("parts", C.c_void_p * 8), ("outs", C.c_void_p * 8),
        ("residual_in", C.c_void_p), ("residual_out", C.c_void_p), ("bias_i32", C.c_void_p),
        ("gamma", C.c_void_p), ("beta", C.c_void_p), ("dq_scale_dev", C.c_void_p),
        ("row_begin", C.c_int64), ("row_count", C.c_int64), ("n", C.c_int64), ("parts_row_begin", C.c_int64),
        ("eps", C.c_float), ("dq_scale", C.c_float), ("world", C.c_int32), ("rank", C.c_int32), ("rounding", C.c_int32),
        ("stream", C.c_void_p),
    ]


_LIB = None


def lib_path() -> str:
    return _build.LIB_PATH


def load():
    """Load (building first if the sources are newer) the CUDA library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_build.LIB_PATH) or (_build.stale() and _build.find_nvcc()):
        _build.build()
    lib = C.CDLL(_build.LIB_PATH)
    lib.ti_gemm_i8.argtypes = [C.POINTER(GemmParams)]
    lib.ti_gemm_i8.restype = C.c_int
    lib.ti_gemm_i8_static_scratch.argtypes = [C.POINTER(GemmParams)]
    lib.ti_gemm_i8_static_scratch.restype = C.c_int
    lib.ti_static_scratch_bytes.restype = C.c_int64
    lib.ti_gemm_workspace_bytes.argtypes = [C.POINTER(GemmParams)]
    lib.ti_gemm_workspace_bytes.restype = C.c_int64
    lib.ti_layernorm.argtypes = [C.POINTER(LayerNormParams)]
    lib.ti_layernorm.restype = C.c_int
    lib.ti_gelu_q.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_float, C.c_int32, C.c_void_p]
    lib.ti_gelu_q.restype = C.c_int
    lib.ti_softmax_q.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int64] * 7 + [C.c_int32, C.c_float, C.c_int32, C.c_void_p]
    lib.ti_softmax_q.restype = C.c_int
    lib.ti_attention_i8.argtypes = [C.POINTER(AttentionParams)]
    lib.ti_attention_i8.restype = C.c_int
    lib.ti_tp_reduce_layernorm_q.argtypes = [C.POINTER(TpReduceLnParams)]
    lib.ti_tp_reduce_layernorm_q.restype = C.c_int
    lib.ti_gemm_i8_scatter.argtypes = [C.POINTER(GemmParams), C.POINTER(GemmScatter)]
    lib.ti_gemm_i8_scatter.restype = C.c_int
    lib.ti_tp_barrier.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_uint32, C.c_void_p]
    lib.ti_tp_barrier.restype = C.c_int
    lib.ti_quantize_absmax.argtypes = [C.POINTER(QuantizeParams)]
    lib.ti_quantize_absmax.restype = C.c_int
    lib.ti_debug_expire_wait.argtypes = [C.c_uint32, C.c_void_p]
    lib.ti_debug_expire_wait.restype = C.c_int
    lib.ti_device_status.argtypes = [C.POINTER(C.c_uint32)]
    lib.ti_device_status.restype = C.c_int
    lib.ti_version.restype = C.c_int
    lib.ti_last_error_string.restype = C.c_char_p
    lib.ti_launch_count.restype = C.c_int64
    lib.ti_device_supported.restype = C.c_int
    _LIB = lib
    return lib


def check(rc: int, what: str):
    """Map a ti_status to the exception type the reference raises for that class of error."""
    if rc == TI_OK:
        return
    msg = f"{what}: {load().ti_last_error_string().decode()} (ti_status {rc})"
    if rc == TI_ERR_SHAPE:
        raise AssertionError(msg)  # the reference's wrappers assert on shape mismatches
    raise RuntimeError(msg)


def device_status() -> int:
    st = C.c_uint32(0)
    rc = load().ti_device_status(C.byref(st))
    if rc not in (TI_OK, TI_ERR_TIMEOUT):
        check(rc, "ti_device_status")
    return st.value


def launch_count() -> int:
    return int(load().ti_launch_count())


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("triton_int_b200 has no CPU path: all tensors must live on a CUDA device")


def current_stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
