"""Offline quantisation helpers with the behaviour of the reference's
functional/quantization.py:5-97 (plain torch; they run once at from_float time
and are not on the hot path).  Like the reference, the ``quantize_*`` and
``fake_quantize_*`` helpers work IN PLACE on their argument where it does."""
import torch


@torch.no_grad()
def quantize_per_tensor_absmax(t):
    scale = t.abs().max() / 127
    if not t.is_cuda:
        t = t.float()  # CPU half tensors cannot round
    t.div_(scale).round_()
    return t.to(torch.int8), scale


@torch.no_grad()
def quantize_weight_per_channel_absmax(w):
    scales = (w.abs().max(dim=1)[0] / 127).view(-1, 1)
    if not w.is_cuda:
        w = w.float()
    w.div_(scales).round_().clamp_(-128, 127)
    return w.to(torch.int8), scales


@torch.no_grad()
def dynamic_quantize_activation_per_tensor_zeropoint(t):
    # the reference indexes a 0-dim max()/min() result ([0]); the scalar is used here
    max_val, min_val = t.max(), t.min()
    nudged_scale = (max_val - min_val) / 254
    zp = (max_val + min_val) / 2
    zp = (zp / nudged_scale).round() * nudged_scale
    t -= zp
    max_val = torch.clamp((max_val - min_val) / 2, min=1e-8) / 127
    q_act = (t / max_val).round().clamp(-128, 127).to(torch.int8)
    return q_act, max_val, zp


@torch.no_grad()
def dynamic_quantize_activation_per_tensor_absmax(t):
    max_val = torch.clamp(t.abs().max(), min=1e-8) / 127
    return (t / max_val).round().clamp(-128, 127).to(torch.int8), max_val


@torch.no_grad()
def dynamic_quantize_activation_per_token_absmax(t):
    max_val = torch.clamp(t.abs().max(dim=-1, keepdim=True)[0], min=1e-8) / 127
    t.div_(max_val).round_().clamp_(-128, 127)
    return t.to(torch.int8), max_val


@torch.no_grad()
def fake_quantize_activation_per_tensor_absmax(t):
    max_val = torch.clamp(t.abs().max(), min=1e-8) / 127
    t.div_(max_val).round_().clamp_(-128, 127).mul_(max_val)
    return t


@torch.no_grad()
def fake_quantize_activation_per_token_absmax(t):
    max_val = torch.clamp(t.abs().max(dim=-1, keepdim=True)[0], min=1e-8) / 127
    t.div_(max_val).round_().clamp_(-128, 127).mul_(max_val)
    return t


@torch.no_grad()
def dequantize_activation_w_per_channel_a_per_token(q_act, w_scales, a_scales):
    out = q_act.to(torch.float32)
    out.mul_(w_scales.reshape(1, -1)).mul_(a_scales.reshape(-1, 1))
    return out.to(a_scales.dtype)


@torch.no_grad()
def dequantize_activation_w_per_channel_a_per_tensor(q_act, w_scales, a_scales):
    out = q_act.to(torch.float32) * w_scales.reshape(1, -1) * a_scales
    return out.to(a_scales.dtype)


# ---------------------------------------------------------------------------
# Fused CUDA forms of the dynamic quantisers (one pass over the activations, input not
# modified).  Same results as the helpers above on CUDA tensors.
def _quantize_cuda(t, per_token, clamp_min):
    import ctypes as C

    from .. import _lib
    _lib.require_cuda(t)
    assert t.dtype in (torch.float32, torch.float16, torch.bfloat16)
    n = t.shape[-1]
    x2 = t.reshape(-1, n)
    if x2.stride(1) != 1 or not per_token:
        x2 = x2.contiguous()
    q = torch.empty(t.shape, dtype=torch.int8, device=t.device)
    p = _lib.QuantizeParams()
    p.x, p.q = x2.data_ptr(), q.data_ptr()
    p.rows, p.n = x2.shape
    p.x_row_stride, p.q_row_stride = x2.stride(0) if x2.shape[0] > 1 else n, n
    p.x_dtype = _lib.DTYPE_CODE[t.dtype]
    p.per_token, p.clamp_min = (1 if per_token else 0), (1 if clamp_min else 0)
    if per_token:
        scales = torch.empty(t.shape[:-1] + (1,), dtype=t.dtype, device=t.device)
    else:
        scales = torch.empty(2, dtype=torch.float32, device=t.device)
    p.scales = scales.data_ptr()
    with torch.cuda.device(t.device):
        p.stream = _lib.current_stream_ptr(t.device)
        rc = _lib.load().ti_quantize_absmax(C.byref(p))
    _lib.check(rc, "ti_quantize_absmax")
    return q, (scales if per_token else scales[0].to(t.dtype))


def dynamic_quantize_activation_per_token_absmax_cuda(t):
    """(int8 tensor, [..., 1] scales): dynamic_quantize_activation_per_token_absmax in one kernel."""
    return _quantize_cuda(t, True, True)


def dynamic_quantize_activation_per_tensor_absmax_cuda(t):
    """(int8 tensor, 0-dim scale): dynamic_quantize_activation_per_tensor_absmax in two kernels."""
    return _quantize_cuda(t, False, True)


def quantize_per_tensor_absmax_cuda(t):
    """(int8 tensor, 0-dim scale): quantize_per_tensor_absmax without touching ``t``."""
    return _quantize_cuda(t, False, False)
