"""LayerNorm-quantise modules.  Reference: torch_int/nn/fused.py:5-43.

``LayerNormQ`` runs as ONE kernel here (the reference issues a cast, a
layer_norm, a round, a clamp and a cast: nn/fused.py:14-17)."""
import torch

from .._CUDA import dq_add_layernorm_q, layernorm_q


class LayerNormQ(torch.nn.Module):
    """int8 = clamp(round(LayerNorm(x) * weight + bias), -128, 127); the output
    scale is folded into weight and bias by ``from_float``."""

    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.input_scale = 1.0
        self.eps = eps
        self.register_buffer("weight", torch.ones(dim, dtype=torch.float32))
        self.register_buffer("bias", torch.zeros(dim, dtype=torch.float32))

    def forward(self, x):
        if x.dtype not in (torch.float32, torch.float16):
            x = x.to(torch.float32)
        elif x.dtype == torch.float16 and self.weight.dtype == torch.float32:
            # The reference casts x to the dtype of the affine parameters first
            # (nn/fused.py:14); fp16 -> fp32 is exact, so the fp16 kernel path with
            # fp32 statistics gives the same result without a cast kernel, except
            # that it would round the LayerNorm output to fp16.  Keep fp32 semantics.
            x = x.to(torch.float32)
        return layernorm_q(x.contiguous(), self.weight, self.bias, self.eps)

    @staticmethod
    def from_float(module: torch.nn.LayerNorm, output_scale: float):
        assert module.normalized_shape[0] == module.weight.numel()
        assert module.normalized_shape[0] == module.bias.numel()
        q = LayerNormQ(module.normalized_shape[0], module.eps)
        q.weight = (module.weight / output_scale).detach().float()
        q.bias = (module.bias / output_scale).detach().float()
        return q


class DQ_Add_LayerNorm_Q(torch.nn.Module):
    """(residual_out, int8) = LayerNormQ(residual + input_scale * int32 input)."""

    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.input_scale = 1.0
        self.eps = eps
        self.register_buffer("weight", torch.ones(dim, dtype=torch.float32))
        self.register_buffer("bias", torch.zeros(dim, dtype=torch.float32))

    def forward(self, residual_input_fp, input_int32):
        return dq_add_layernorm_q(input_int32, self.input_scale, residual_input_fp,
                                  self.weight, self.bias, self.eps)
