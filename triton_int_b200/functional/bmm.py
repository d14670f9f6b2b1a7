"""Functional aliases of the attention BMMs (reference functional/bmm.py:6-18)."""
from ..kernels.bmm import bmm_s8t_s8n_s8t, bmm_s8t_s8n_s32t


def bmm_i8_o8(a, b, scale):
    """int8 [B,M,N] = int8(scale * a[B,M,K] . b[B,N,K]^T)."""
    return bmm_s8t_s8n_s8t(a, b, scale)


def bmm_i8_o32(a, b):
    """int32 [B,M,N] = a[B,M,K] . b[B,N,K]^T."""
    return bmm_s8t_s8n_s32t(a, b)
