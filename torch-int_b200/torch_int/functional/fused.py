"""dequant + residual add + LayerNorm + quantise (torch_int/functional/fused.py:5-25)."""
import torch

from torch_int._CUDA import dq_add_layernorm_q


def dq_add_layernorm_q_py(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """Unfused torch formulation of the op, kept for comparison (functional/fused.py:5-12)."""
    residual = torch.add(residual_input_fp, input_int32, alpha=input_scale_fp)
    ln = torch.nn.functional.layer_norm(residual, residual.shape[-1:], gamma, beta, eps)
    return residual, ln.clamp(-128, 127).round().to(torch.int8)


def dq_add_layernorm(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """As above without the final quantisation (functional/fused.py:15-21)."""
    residual = torch.add(residual_input_fp, input_int32, alpha=input_scale_fp)
    return residual, torch.nn.functional.layer_norm(residual, residual.shape[-1:], gamma, beta, eps)


def dq_add_layernorm_q_cpp(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps):
    """The native fused kernel (functional/fused.py:24-25)."""
    return dq_add_layernorm_q(input_int32, input_scale_fp, residual_input_fp, gamma, beta, eps)
