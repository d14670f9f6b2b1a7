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
