"""LayerNorm-quantise modules.  Reference: torch_int/nn/fused.py:5-43.

``LayerNormQ`` runs as ONE kernel here (the reference issues a cast, a
layer_norm, a round, a clamp and a cast: nn/fused.py:14-17)."""
import torch

from .._CUDA import dq_add_layernorm_q, layernorm_q


class _QuantisingNorm(torch.nn.Module):
    """State shared by both modules, with the reference's names: fp32 buffers ``weight`` and ``bias``
    of the affine step (the output scale already divided in), ``eps`` and ``input_scale``."""

    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.input_scale = 1.0
        for name, fill in (("weight", 1.0), ("bias", 0.0)):
            self.register_buffer(name, torch.full((dim,), fill, dtype=torch.float32))


class LayerNormQ(_QuantisingNorm):
    """int8 = clamp(round(LayerNorm(x) * weight + bias), -128, 127); the output
    scale is folded into weight and bias by ``from_float``."""

    def forward(self, x):
        # The reference casts x to the dtype of the affine parameters first (nn/fused.py:14), normally
        # fp32, and normalises there; only when the parameters themselves were cast to fp16 is the
        # LayerNorm output an fp16 tensor.  fp16 inputs are read as they are (no widening copy): the
        # kernel converts on load.
        half_params = self.weight.dtype == torch.float16
        if x.dtype not in (torch.float32, torch.float16):
            x = x.to(torch.float32)
        if x.dtype == torch.float16:
            return layernorm_q(x.contiguous(), self.weight, self.bias, self.eps, fp32_norm=not half_params)
        return layernorm_q(x.contiguous(), self.weight, self.bias, self.eps)

    @staticmethod
    def from_float(module: torch.nn.LayerNorm, output_scale: float):
        dim = module.normalized_shape[0]
        if module.weight.numel() != dim or module.bias.numel() != dim:
            raise AssertionError("LayerNormQ.from_float needs a one-dimensional affine LayerNorm")
        q = LayerNormQ(dim, module.eps)
        q.weight = (module.weight / output_scale).detach().float()
        q.bias = (module.bias / output_scale).detach().float()
        return q


class DQ_Add_LayerNorm_Q(_QuantisingNorm):
    """(residual_out, int8) = LayerNormQ(residual + input_scale * int32 input)."""

    def forward(self, residual_input_fp, input_int32):
        return dq_add_layernorm_q(input_int32, self.input_scale, residual_input_fp,
                                  self.weight, self.bias, self.eps)
