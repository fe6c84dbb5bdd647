"""Aliases of the batched int8 products (torch_int/functional/bmm.py:5-17)."""
from torch_int._CUDA import bmm_s8t_s8n_s8t, bmm_s8t_s8n_s32t


def bmm_i8_o8(a, b, scale):
    """int8 [B,M,N] = sat_rne(scale * a[b] . b[b]^T) for int8 a [B,M,K], b [B,N,K]."""
    return bmm_s8t_s8n_s8t(a, b, scale)


def bmm_i8_o32(a, b):
    """int32 [B,M,N] = a[b] . b[b]^T."""
    return bmm_s8t_s8n_s32t(a, b)
