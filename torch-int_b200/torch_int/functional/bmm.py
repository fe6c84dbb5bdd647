"""Short names for two of the batched int8 products (torch_int/functional/bmm.py:5-17 of the reference).

Operands are int8 ``a`` [B, M, K] and ``b`` [B, N, K]; the product is a[i] . b[i]^T per batch entry.
"""
from torch_int import _CUDA as _ops


def bmm_i8_o8(a, b, scale):
    """int8 [B, M, N]: the int32 product scaled by ``scale``, rounded half to even and saturated."""
    return _ops.bmm_s8t_s8n_s8t(a, b, scale)


def bmm_i8_o32(a, b):
    """int32 [B, M, N]: the exact product."""
    return _ops.bmm_s8t_s8n_s32t(a, b)
