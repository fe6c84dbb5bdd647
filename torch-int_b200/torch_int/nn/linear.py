"""W8A8 linear modules: int8 weight [out,in], per-tensor scales folded into two
scalars.  Class names, constructor signatures, buffer names/shapes/dtypes and
``from_float`` follow torch_int/nn/linear.py so that checkpoints exported for
the reference load unchanged.

Unlike the reference forwards (nn/linear.py:41,85,157,214) the scalar buffers
are not read back with ``.item()`` on every call: the Python floats are cached
and refreshed only when the buffer object or its version counter changes, so a
forward pass does not synchronise the device.
"""
import torch

from .._CUDA import (linear_a8_w8_b8_o8, linear_a8_w8_b32_o32, linear_a8_w8_b32_o32_with_scaling,
                     linear_a8_w8_bfp32_ofp32, linear_relu_a8_w8_b8_o8)
from ..functional.quantization import (fake_quantize_activation_per_tensor_absmax,
                                       fake_quantize_activation_per_token_absmax,
                                       quantize_per_tensor_absmax,
                                       quantize_weight_per_channel_absmax)


class _W8A8Base(torch.nn.Module):
    """Shared plumbing: buffers, ``to``, flatten -> op -> unflatten."""

    _bias_dtype = torch.int8
    _has_beta = True

    def __init__(self, in_features, out_features, alpha=1.0, beta=1.0):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        # Same default initialisation as the reference (nn/linear.py:23-28).
        self.register_buffer("weight", torch.randint(-127, 127, (out_features, in_features),
                                                     dtype=torch.int8, requires_grad=False))
        self.register_buffer("bias", torch.zeros((1, out_features), dtype=self._bias_dtype,
                                                 requires_grad=False))
        if alpha is not None:
            self.register_buffer("a", torch.tensor(alpha))
        if self._has_beta and beta is not None:
            self.register_buffer("b", torch.tensor(beta))
        self._scalars = {}

    def to(self, *args, **kwargs):
        # Integer buffers are untouched by dtype casts but must follow device moves
        # (nn/linear.py:30-34).
        super().to(*args, **kwargs)
        self.weight = self.weight.to(*args, **kwargs)
        self.bias = self.bias.to(*args, **kwargs)
        return self

    def _scalar(self, name):
        t = getattr(self, name)
        if not torch.is_tensor(t):
            return float(t)
        hit = self._scalars.get(name)
        if hit is not None and hit[0] is t and hit[1] == t._version:
            return hit[2]
        v = float(t.item())
        self._scalars[name] = (t, t._version, v)
        return v

    def _op(self, x2d):
        raise NotImplementedError

    @torch.no_grad()
    def forward(self, x):
        shape = x.shape
        y = self._op(x.view(-1, shape[-1]))
        return y.view(*shape[:-1], -1)

    @classmethod
    def _from_float_int8_bias(cls, module, input_scale, output_scale):
        q = cls(module.in_features, module.out_features)
        w8, w_scale = quantize_per_tensor_absmax(module.weight)
        b8, b_scale = quantize_per_tensor_absmax(module.bias)
        q.weight = w8
        q.bias = b8
        q.a = input_scale * w_scale / output_scale
        q.b = b_scale / output_scale
        return q


class W8A8B8O8Linear(_W8A8Base):
    """int8 in, int8 weight, int8 bias, int8 out (q/k/v projections).
    Reference: torch_int/nn/linear.py:16-57."""

    def _op(self, x2d):
        return linear_a8_w8_b8_o8(x2d, self.weight, self.bias, self._scalar("a"), self._scalar("b"))

    @staticmethod
    def from_float(module: torch.nn.Linear, input_scale, output_scale):
        return W8A8B8O8Linear._from_float_int8_bias(module, input_scale, output_scale)


class W8A8B8O8LinearReLU(_W8A8Base):
    """As W8A8B8O8Linear with a fused ReLU (fc1).  Reference: nn/linear.py:60-102."""

    def _op(self, x2d):
        return linear_relu_a8_w8_b8_o8(x2d, self.weight, self.bias, self._scalar("a"), self._scalar("b"))

    @staticmethod
    def from_float(module: torch.nn.Linear, input_scale, output_scale):
        return W8A8B8O8LinearReLU._from_float_int8_bias(module, input_scale, output_scale)


class W8A8B32O32LinearWithoutScaling(_W8A8Base):
    """int32 out = x . W^T + int32 bias, no scaling.  Reference: nn/linear.py:105-129."""

    _bias_dtype = torch.int32

    def __init__(self, in_features, out_features):
        super().__init__(in_features, out_features, alpha=None, beta=None)

    def _op(self, x2d):
        return linear_a8_w8_b32_o32(x2d, self.weight, self.bias)


class W8A8B32O32Linear(_W8A8Base):
    """int32 out = rne(alpha * x . W^T + beta * int32 bias).  Reference: nn/linear.py:132-179."""

    _bias_dtype = torch.int32

    def _op(self, x2d):
        return linear_a8_w8_b32_o32_with_scaling(x2d, self.weight, self.bias,
                                                 self._scalar("a"), self._scalar("b"))

    @staticmethod
    def from_float(module: torch.nn.Linear, input_scale, output_scale):
        q = W8A8B32O32Linear(module.in_features, module.out_features)
        w8, w_scale = quantize_per_tensor_absmax(module.weight)
        bias = module.bias.float()
        b_scale = bias.abs().max() / (2 ** 31 - 1)
        q.weight = w8
        q.bias = (bias / b_scale).round().to(torch.int32)
        q.a = input_scale * w_scale / output_scale
        q.b = b_scale / output_scale
        q.input_scale, q.output_scale = input_scale, output_scale
        q.weight_scale, q.bias_scale = w_scale, b_scale
        return q


class W8A8BFP32OFP32Linear(_W8A8Base):
    """fp32 out = alpha * x . W^T + fp32 bias (out_proj, fc2).  The bias stays fp32
    under ``.half()`` / dtype casts.  Reference: nn/linear.py:182-229."""

    _bias_dtype = torch.float32
    _has_beta = False

    def _apply(self, fn, *args, **kwargs):
        super()._apply(fn, *args, **kwargs)
        self.bias = self.bias.to(torch.float32)
        return self

    def to(self, *args, **kwargs):
        super().to(*args, **kwargs)
        self.bias = self.bias.to(torch.float32)
        return self

    def _op(self, x2d):
        if self.bias.dtype != torch.float32:
            self.bias = self.bias.to(torch.float32)
        return linear_a8_w8_bfp32_ofp32(x2d, self.weight, self.bias, self._scalar("a"), 1)

    @staticmethod
    def from_float(module: torch.nn.Linear, input_scale):
        q = W8A8BFP32OFP32Linear(module.in_features, module.out_features)
        w8, w_scale = quantize_per_tensor_absmax(module.weight)
        q.weight = w8
        q.bias = module.bias.detach().to(torch.float32).reshape(1, -1)
        q.a = input_scale * w_scale
        q.input_scale, q.weight_scale = input_scale, w_scale
        return q


class _W8FloatActBase(torch.nn.Module):
    """int8 weights de-quantised to fp16 on the fly; activations stay floating
    point.  Pure PyTorch simulation modules, not W8A8 kernels."""

    def __init__(self, in_features, out_features, bias=True):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.register_buffer("weight", torch.randint(-127, 127, (out_features, in_features),
                                                     dtype=torch.int8, requires_grad=False))
        self.register_buffer("bias", torch.zeros((1, out_features), dtype=torch.float16,
                                                 requires_grad=False) if bias else None)
        self.register_buffer("weight_scales", torch.ones(out_features, dtype=torch.float16,
                                                         requires_grad=False))

    def to(self, *args, **kwargs):
        super().to(*args, **kwargs)
        self.weight = self.weight.to(*args, **kwargs)
        if self.bias is not None:
            self.bias = self.bias.to(*args, **kwargs)
        self.weight_scales = self.weight_scales.to(*args, **kwargs)
        return self

    def __repr__(self):
        return super().__repr__() + f"({self.in_features}, {self.out_features}, bias={self.bias is not None})"


class W8A16Linear(_W8FloatActBase):
    """fp16 activations x de-quantised int8 weights.  Reference: nn/linear.py:232-282."""

    @torch.no_grad()
    def forward(self, x):
        w = self.weight.to(torch.float16) * self.weight_scales
        return torch.nn.functional.linear(x, w, self.bias)

    @staticmethod
    def from_float(module, weight_quant="per_channel"):
        assert isinstance(module, torch.nn.Linear)
        q = W8A16Linear(module.in_features, module.out_features, module.bias is not None)
        if weight_quant == "per_channel":
            q.weight, q.weight_scales = quantize_weight_per_channel_absmax(module.weight)
        elif weight_quant == "per_tensor":
            q.weight, q.weight_scales = quantize_per_tensor_absmax(module.weight)
        else:
            raise ValueError('weight_quant must be "per_channel" or "per_tensor"')
        if module.bias is not None:
            q.bias = module.bias.to(torch.float16)
        return q


class W8FakeA8Linear(_W8FloatActBase):
    """Fake-quantised activations x de-quantised int8 weights.  Reference: nn/linear.py:285-337."""

    def __init__(self, in_features, out_features, bias=True, act_quant="per_token"):
        super().__init__(in_features, out_features, bias)
        if act_quant == "per_token":
            self.activation_fake_quantizer = fake_quantize_activation_per_token_absmax
        elif act_quant == "per_tensor":
            self.activation_fake_quantizer = fake_quantize_activation_per_tensor_absmax
        else:
            raise ValueError('act_quant must be "per_token" or "per_tensor"')

    @torch.no_grad()
    def forward(self, x):
        w = self.weight.to(torch.float16) * self.weight_scales.view(-1, 1)
        return torch.nn.functional.linear(self.activation_fake_quantizer(x), w, self.bias)

    @staticmethod
    def from_float(module, act_quant="per_token"):
        assert isinstance(module, torch.nn.Linear)
        q = W8FakeA8Linear(module.in_features, module.out_features, module.bias is not None, act_quant)
        q.weight, q.weight_scales = quantize_weight_per_channel_absmax(module.weight)
        if module.bias is not None:
            q.bias = module.bias.to(torch.float16)
        return q
