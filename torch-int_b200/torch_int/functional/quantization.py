"""Absmax quantisers used when converting float modules (offline, not timed).

Same names and results as torch_int/functional/quantization.py; unlike the
reference (quantization.py:12,25) the source tensor is NOT modified in place.
"""
import torch


@torch.no_grad()
def quantize_per_tensor_absmax(t):
    """(int8 tensor, scale) with scale = max|t| / 127 (quantization.py:6-14)."""
    scale = t.abs().max() / 127
    q = (t.float() / scale.float()).round() if not t.is_cuda else (t / scale).round()
    return q.to(torch.int8), scale


@torch.no_grad()
def quantize_weight_per_channel_absmax(w):
    """(int8 [out,in], scales [out,1]) with one scale per output row (quantization.py:17-27)."""
    scales = (w.abs().max(dim=1)[0] / 127).view(-1, 1)
    q = (w.float() / scales.float()) if not w.is_cuda else (w / scales)
    return q.round().clamp(-128, 127).to(torch.int8), scales


@torch.no_grad()
def dynamic_quantize_activation_per_tensor_absmax(t):
    """(int8, scale) with a scale computed from this tensor (quantization.py:48-52)."""
    scale = torch.clamp(t.abs().max(), min=1e-8) / 127
    return (t / scale).round().clamp(-128, 127).to(torch.int8), scale


@torch.no_grad()
def dynamic_quantize_activation_per_token_absmax(t):
    """(int8, scales [..., 1]) with one scale per row of the last dimension (quantization.py:55-61)."""
    scale = torch.clamp(t.abs().max(dim=-1, keepdim=True)[0], min=1e-8) / 127
    return (t / scale).round().clamp(-128, 127).to(torch.int8), scale


@torch.no_grad()
def fake_quantize_activation_per_tensor_absmax(t):
    """Quantise-dequantise with one scale; returns a float tensor (quantization.py:63-68)."""
    scale = torch.clamp(t.abs().max(), min=1e-8) / 127
    return (t / scale).round().clamp(-128, 127) * scale


@torch.no_grad()
def fake_quantize_activation_per_token_absmax(t):
    """Quantise-dequantise with one scale per row (quantization.py:71-76)."""
    scale = torch.clamp(t.abs().max(dim=-1, keepdim=True)[0], min=1e-8) / 127
    return (t / scale).round().clamp(-128, 127) * scale


@torch.no_grad()
def dequantize_activation_w_per_channel_a_per_token(q_act, w_scales, a_scales):
    """int accumulators [B,dim] * w_scales[dim] * a_scales[B,1] (quantization.py:79-87)."""
    out = q_act.to(torch.float32) * w_scales.reshape(1, -1) * a_scales.reshape(-1, 1)
    return out.to(a_scales.dtype)


@torch.no_grad()
def dequantize_activation_w_per_channel_a_per_tensor(q_act, w_scales, a_scales):
    """int accumulators [...,dim] * w_scales[dim] * a_scales[1] (quantization.py:89-97)."""
    out = q_act.to(torch.float32) * w_scales.reshape(1, -1) * a_scales
    return out.to(a_scales.dtype)
