"""Functional forms of dequantise + residual add + LayerNorm (+ quantise).

Same names and argument order as torch_int/functional/fused.py:5-25 of the reference:
``dq_add_layernorm_q_cpp`` is the native one-kernel op, ``dq_add_layernorm_q_py`` and
``dq_add_layernorm`` are the plain-torch formulations the reference keeps beside it for
comparison (they work on any device).
"""
import torch
import torch.nn.functional as F

from torch_int import _CUDA as _ops


def dq_add_layernorm(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """(residual + scale * int32 input, LayerNorm of that over the last dimension), in floating point."""
    summed = torch.add(residual_input_fp, input_int32, alpha=input_scale_fp)
    return summed, F.layer_norm(summed, summed.shape[-1:], gamma, beta, eps)


def dq_add_layernorm_q_py(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """dq_add_layernorm followed by clamp to [-128, 127], round half to even and a cast to int8."""
    summed, normed = dq_add_layernorm(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps)
    return summed, normed.clamp(-128, 127).round().to(torch.int8)


def dq_add_layernorm_q_cpp(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """The same result from the fused CUDA kernel (one pass over the row)."""
    return _ops.dq_add_layernorm_q(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps)
