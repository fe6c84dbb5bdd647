"""Absmax quantisers used when converting float modules (offline, not timed).

Same names and results as torch_int/functional/quantization.py of the reference; unlike the reference
(quantization.py:12,25,58,66,74) no function modifies its argument in place.  All of them are built from two
steps: a scale = max|t| / 127 (over the whole tensor, per output row of a weight, or per token), and
round-half-to-even of t / scale into the int8 range.
"""
import torch

_QMAX = 127


def _scale(t, dim=None, floor=None):
    """max|t| / 127 over everything (dim=None) or over `dim` (kept); `floor` guards all-zero inputs."""
    peak = t.abs().max() if dim is None else t.abs().max(dim=dim, keepdim=True)[0]
    if floor is not None:
        peak = torch.clamp(peak, min=floor)
    return peak / _QMAX


def _grid(t, scale, clamp=True):
    """t / scale rounded half to even (in fp32 on CPU, where half-precision rounding is unavailable)."""
    if not t.is_cuda and t.dtype in (torch.float16, torch.bfloat16):
        t, scale = t.float(), scale.float()
    q = (t / scale).round()
    return q.clamp(-128, _QMAX) if clamp else q


@torch.no_grad()
def quantize_per_tensor_absmax(t):
    """(int8 tensor, scale) with one scale for the tensor (quantization.py:6-14)."""
    scale = _scale(t)
    return _grid(t, scale, clamp=False).to(torch.int8), scale


@torch.no_grad()
def quantize_weight_per_channel_absmax(w):
    """(int8 [out, in], scales [out, 1]) with one scale per output row (quantization.py:17-27)."""
    scales = _scale(w, dim=1)
    return _grid(w, scales).to(torch.int8), scales


@torch.no_grad()
def dynamic_quantize_activation_per_tensor_absmax(t):
    """(int8, scale) with a scale computed from this tensor (quantization.py:48-52)."""
    scale = _scale(t, floor=1e-8)
    return _grid(t, scale).to(torch.int8), scale


@torch.no_grad()
def dynamic_quantize_activation_per_token_absmax(t):
    """(int8, scales [..., 1]) with one scale per row of the last dimension (quantization.py:55-61)."""
    scale = _scale(t, dim=-1, floor=1e-8)
    return _grid(t, scale).to(torch.int8), scale


@torch.no_grad()
def fake_quantize_activation_per_tensor_absmax(t):
    """Quantise-dequantise with one scale; returns a float tensor (quantization.py:63-68)."""
    scale = _scale(t, floor=1e-8)
    return _grid(t, scale) * scale


@torch.no_grad()
def fake_quantize_activation_per_token_absmax(t):
    """Quantise-dequantise with one scale per row (quantization.py:71-76)."""
    scale = _scale(t, dim=-1, floor=1e-8)
    return _grid(t, scale) * scale


def _dequantize(q_act, w_scales, a_scales):
    out = q_act.to(torch.float32) * w_scales.reshape(1, -1) * a_scales
    return out.to(a_scales.dtype)


@torch.no_grad()
def dequantize_activation_w_per_channel_a_per_token(q_act, w_scales, a_scales):
    """int accumulators [B, dim] * w_scales[dim] * a_scales[B, 1] (quantization.py:79-87)."""
    return _dequantize(q_act, w_scales, a_scales.reshape(-1, 1))


@torch.no_grad()
def dequantize_activation_w_per_channel_a_per_tensor(q_act, w_scales, a_scales):
    """int accumulators [..., dim] * w_scales[dim] * a_scales[1] (quantization.py:89-97)."""
    return _dequantize(q_act, w_scales, a_scales)
