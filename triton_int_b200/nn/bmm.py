"""Attention BMM modules (reference nn/bmm.py:10-130): one 0-dim scale buffer
``a`` each, ``forward(a, b)`` on 3-D int8 tensors, ``from_scale`` constructors."""
from __future__ import annotations

import torch

from ..kernels.bmm import bmm_s8t_s8n_f32t, bmm_s8t_s8n_s8t, bmm_s8t_s8n_s32t, bmm_s8t_s8t_s8t


def _as_tensor(alpha):
    return alpha if torch.is_tensor(alpha) else torch.tensor(alpha)


class _ScaledBMM(torch.nn.Module):
    def __init__(self, alpha):
        super().__init__()
        self.register_buffer("a", torch.tensor(alpha))


class BMM_S8T_S8N_S8T(_ScaledBMM):
    """a [B,M,K] int8, b [B,N,K] int8 -> int8 [B,M,N] (reference nn/bmm.py:10-29)."""

    @torch.no_grad()
    def forward(self, a, b):
        return bmm_s8t_s8n_s8t(a, b, self.a)

    @classmethod
    def from_scale(cls, a_scale, b_scale, output_scale):
        m = cls(1.0)
        m.a = _as_tensor(a_scale * b_scale / output_scale)
        return m


class BMM_S8T_S8T_S8T(_ScaledBMM):
    """a [B,M,K] int8, b [B,K,N] int8 -> int8 [B,M,N] (reference nn/bmm.py:32-51)."""

    @torch.no_grad()
    def forward(self, a, b):
        return bmm_s8t_s8t_s8t(a, b, self.a)

    @classmethod
    def from_scale(cls, a_scale, b_scale, output_scale):
        m = cls(1.0)
        m.a = _as_tensor(a_scale * b_scale / output_scale)
        return m


class BMM_S8T_S8N_F32T(_ScaledBMM):
    """a [B,M,K], b [B,N,K] -> floating [B,M,N] (reference nn/bmm.py:54-74)."""

    def __init__(self, alpha, dtype=torch.float32):
        super().__init__(alpha)
        self.dtype = dtype

    @torch.no_grad()
    def forward(self, a, b):
        return bmm_s8t_s8n_f32t(a, b, self.a, dtype=self.dtype)

    @classmethod
    def from_scale(cls, a_scale, b_scale, dtype=torch.float32):
        m = cls(1.0, dtype=dtype)
        m.a = _as_tensor(a_scale * b_scale)
        return m


class BMM_S8T_S8N_F16T(BMM_S8T_S8N_F32T):
    """fp16 output (reference nn/bmm.py:77-96)."""

    def __init__(self, alpha):
        super().__init__(alpha, torch.float16)

    @classmethod
    def from_scale(cls, a_scale, b_scale):
        m = cls(1.0)
        m.a = _as_tensor(a_scale * b_scale)
        return m


class BMM_S8T_S8N_BF16T(BMM_S8T_S8N_F16T):
    """bf16 output (reference nn/bmm.py:99-118)."""

    def __init__(self, alpha):
        BMM_S8T_S8N_F32T.__init__(self, alpha, torch.bfloat16)


class BMM_S8T_S8N_S32T(torch.nn.Module):
    """Raw int32 accumulators (reference nn/bmm.py:121-130)."""

    @torch.no_grad()
    def forward(self, a, b):
        return bmm_s8t_s8n_s32t(a, b)
