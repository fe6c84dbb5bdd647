"""Host-side behaviour of the torch_int package that needs no GPU: module
surface, buffer names, from_float arithmetic, and loud failure without CUDA."""
import pytest
import torch

import torch_int  # noqa: F401
from torch_int import _CUDA
from torch_int.nn.bmm import BMM_S8T_S8N_F32T, BMM_S8T_S8N_S8T, BMM_S8T_S8N_S32T
from torch_int.nn.fused import DQ_Add_LayerNorm_Q, LayerNormQ
from torch_int.nn.linear import (W8A8B8O8Linear, W8A8B8O8LinearReLU, W8A8B32O32Linear,
                                 W8A8B32O32LinearWithoutScaling, W8A8BFP32OFP32Linear, W8A16Linear,
                                 W8FakeA8Linear)


def test_reference_callables_exist():
    # torch_int/kernels/bindings.cpp:5-20
    for name in ("linear_relu_a8_w8_b8_o8", "linear_a8_w8_b32_o32", "linear_a8_w8_bfp32_ofp32",
                 "linear_a8_w8_b32_o32_with_scaling", "linear_a8_w8_b8_o8", "dq_add_layernorm_q",
                 "bmm_s8t_s8n_s8t", "bmm_s8t_s8n_f32t", "bmm_s8t_s8n_s32t"):
        assert callable(getattr(_CUDA, name))
    assert torch_int.nn.W8A16Linear is W8A16Linear and torch_int.nn.W8FakeA8Linear is W8FakeA8Linear


def test_buffer_names_shapes_dtypes():
    # torch_int/nn/linear.py:23-28,112-115,189-193; nn/bmm.py:8; nn/fused.py:10-11
    m = W8A8B8O8Linear(32, 48, alpha=0.5, beta=0.25)
    sd = m.state_dict()
    assert list(sd) == ["weight", "bias", "a", "b"]
    assert sd["weight"].shape == (48, 32) and sd["weight"].dtype == torch.int8
    assert sd["bias"].shape == (1, 48) and sd["bias"].dtype == torch.int8
    assert sd["a"].dim() == 0 and float(sd["a"]) == 0.5 and float(sd["b"]) == 0.25
    assert list(W8A8B8O8LinearReLU(32, 48).state_dict()) == ["weight", "bias", "a", "b"]
    assert list(W8A8B32O32LinearWithoutScaling(32, 48).state_dict()) == ["weight", "bias"]
    assert W8A8B32O32Linear(32, 48).bias.dtype == torch.int32
    f = W8A8BFP32OFP32Linear(32, 48)
    assert list(f.state_dict()) == ["weight", "bias", "a"] and f.bias.dtype == torch.float32
    f.half()
    assert f.bias.dtype == torch.float32, "the fp32 bias must survive .half() (nn/linear.py:195-206)"
    assert list(BMM_S8T_S8N_S8T(1.0).state_dict()) == ["a"]
    assert list(BMM_S8T_S8N_S32T().state_dict()) == []
    assert list(LayerNormQ(8).state_dict()) == ["weight", "bias"]
    assert list(DQ_Add_LayerNorm_Q(8).state_dict()) == ["weight", "bias"]
    assert W8A16Linear(8, 4).weight_scales.dtype == torch.float16
    assert W8FakeA8Linear(8, 4, act_quant="per_tensor").bias.shape == (1, 4)


def test_from_float_scale_folding_and_no_mutation():
    torch.manual_seed(0)
    lin = torch.nn.Linear(64, 32)
    w0, b0 = lin.weight.detach().clone(), lin.bias.detach().clone()
    q = W8A8B8O8Linear.from_float(lin, input_scale=0.02, output_scale=0.05)
    assert torch.equal(lin.weight, w0) and torch.equal(lin.bias, b0), "from_float must not modify the float module"
    ws = w0.abs().max() / 127
    bs = b0.abs().max() / 127
    assert torch.equal(q.weight, (w0 / ws).round().to(torch.int8))          # nn/linear.py:49
    assert torch.allclose(q.a, 0.02 * ws / 0.05) and torch.allclose(q.b, bs / 0.05)  # :51-52
    q = W8A8BFP32OFP32Linear.from_float(lin, input_scale=0.02)
    assert torch.allclose(q.a, 0.02 * ws) and torch.equal(q.bias.reshape(-1), b0)   # :224-226
    q = W8A8B32O32Linear.from_float(lin, 0.02, 0.05)
    assert q.bias.dtype == torch.int32 and torch.allclose(q.b, (b0.abs().max() / (2 ** 31 - 1)) / 0.05)
    ln = torch.nn.LayerNorm(64)
    ln.weight.data.uniform_(0.5, 1.5)
    lq = LayerNormQ.from_float(ln, 0.1)
    assert torch.allclose(lq.weight, ln.weight / 0.1) and lq.eps == ln.eps           # nn/fused.py:24-26
    bm = BMM_S8T_S8N_S8T.from_scale(0.1, 0.2, 0.4)
    assert abs(float(bm.a) - 0.05) < 1e-7                                            # nn/bmm.py:19-23
    bm = BMM_S8T_S8N_F32T.from_scale(torch.tensor(0.1), 0.2)
    assert abs(float(bm.a) - 0.02) < 1e-7


def test_scalar_cache_follows_buffer_updates():
    m = W8A8B8O8Linear(16, 16, alpha=2.0, beta=3.0)
    assert m._scalar("a") == 2.0
    m.a = torch.tensor(5.0)
    assert m._scalar("a") == 5.0
    m.a.fill_(7.0)
    assert m._scalar("a") == 7.0
    m.load_state_dict({**m.state_dict(), "a": torch.tensor(9.0)})
    assert m._scalar("a") == 9.0


def test_no_cpu_fallback():
    """The product must fail loudly, not compute on the CPU."""
    x = torch.zeros((4, 16), dtype=torch.int8)
    w = torch.zeros((16, 16), dtype=torch.int8)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _CUDA.linear_a8_w8_b8_o8(x, w, torch.zeros(16, dtype=torch.int8), 1.0, 1.0)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _CUDA.bmm_s8t_s8n_s32t(x[None], w[None])
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        W8A8B8O8Linear(16, 16)(x)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        LayerNormQ(16)(torch.zeros(2, 16))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _CUDA.dq_add_layernorm_q(torch.zeros((2, 16), dtype=torch.int32), 0.1, torch.zeros(2, 16),
                                 torch.ones(16), torch.zeros(16), 1e-5)


def test_lm_head_logits_helper_on_cpu():
    """Int8OPTForCausalLM._logits is plain torch: tied table, cast to the table's dtype, and the
    vocabulary-parallel form only when a tensor-parallel context asks for it."""
    from torch_int.models.opt import Int8OPTConfig
    from torch_int.models.random_init import random_int8_opt
    cfg = Int8OPTConfig(vocab_size=48, hidden_size=32, num_hidden_layers=1, ffn_dim=64, num_attention_heads=2,
                        max_position_embeddings=16)
    model = random_int8_opt(cfg, seed=1, device="cpu")
    hidden = torch.randn(2, 3, 32, generator=torch.Generator().manual_seed(2))
    want = torch.nn.functional.linear(hidden, model.model.decoder.embed_tokens.weight)
    assert torch.equal(model._logits(hidden), want)
    assert torch.equal(model._logits(hidden.double()), want)          # cast to the table's dtype first
    attn = model.model.decoder.layers[0].self_attn
    assert attn.fused_attention is True                               # one-kernel causal attention is the default


def test_from_float_matches_the_reference_modules(golden_dir):
    """from_float / from_scale of the modules here against the results of the REFERENCE's own conversion
    code on the same seeded float modules (tests/golden/from_float.npz, made by make_golden.py): quantised
    weights and biases identical, scale factors equal to fp32 rounding, and the float module untouched
    (the reference quantises its argument in place, functional/quantization.py:12)."""
    import os
    import numpy as np
    from torch_int.nn.bmm import BMM_S8T_S8N_F32T, BMM_S8T_S8N_S8T
    from torch_int.nn.fused import LayerNormQ
    from torch_int.nn.linear import W8A8B8O8Linear, W8A8B8O8LinearReLU, W8A8B32O32Linear, W8A8BFP32OFP32Linear
    z = np.load(os.path.join(golden_dir, "from_float.npz"))
    lin = torch.nn.Linear(48, 80)
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(z["w"]))
        lin.bias.copy_(torch.from_numpy(z["b"]))
    s_in, s_out = float(z["input_scale"]), float(z["output_scale"])

    def close(a, b):
        return abs(float(a) - float(b)) <= 2e-7 * abs(float(b))

    for tag, cls in (("b8o8", W8A8B8O8Linear), ("relu", W8A8B8O8LinearReLU), ("b32o32", W8A8B32O32Linear)):
        m = cls.from_float(lin, s_in, s_out)
        assert np.array_equal(m.weight.numpy(), z[f"{tag}_weight"]), tag
        assert np.array_equal(m.bias.numpy().reshape(-1), z[f"{tag}_bias"].reshape(-1)), tag
        assert m.bias.dtype == torch.from_numpy(z[f"{tag}_bias"]).dtype
        assert close(m._scalar("a"), z[f"{tag}_a"]) and close(m._scalar("b"), z[f"{tag}_b"]), tag
    m = W8A8BFP32OFP32Linear.from_float(lin, s_in)
    assert np.array_equal(m.weight.numpy(), z["bfp32_weight"])
    assert np.array_equal(m.bias.numpy().reshape(-1), z["bfp32_bias"].reshape(-1)) and m.bias.dtype == torch.float32
    assert close(m._scalar("a"), z["bfp32_a"])
    assert np.array_equal(lin.weight.detach().numpy(), z["w"]) and np.array_equal(lin.bias.detach().numpy(), z["b"])
    assert close(BMM_S8T_S8N_S8T.from_scale(1.0 / 127, 0.031, 0.044)._alpha(), z["bmm_s8t_a"])
    assert close(BMM_S8T_S8N_F32T.from_scale(0.021, 0.017)._alpha(), z["bmm_f32t_a"])
    ln = torch.nn.LayerNorm(96)
    with torch.no_grad():
        ln.weight.copy_(torch.from_numpy(z["ln_w"]))
        ln.bias.copy_(torch.from_numpy(z["ln_b"]))
    q = LayerNormQ.from_float(ln, float(z["ln_output_scale"]))
    assert np.array_equal(q.weight.numpy(), z["lnq_weight"]) and np.array_equal(q.bias.numpy(), z["lnq_bias"])
    assert q.eps == float(z["ln_eps"])


@pytest.mark.gpu
def test_status_reset_clears_the_split_k_workspace(monkeypatch):
    """A launch that gave up on a bounded wait may leave partial sums in the split-K scratch, which every later
    small-M GEMM expects all zero: device_status(reset=True) must hand it back zeroed together with the status
    word.  The non-zero status is injected on the host (no kernel is made to time out)."""
    from torch_int import _CUDA as C
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = C._split_k_workspace(dev)
    ws[:4096].fill_(7)
    real = C._c_device_status

    def fake(status_ptr, reset):
        real(status_ptr, reset)
        status_ptr._obj.value = 105          # byref(c_int) -> the c_int the caller reads afterwards
        return 0
    monkeypatch.setattr(C, "_c_device_status", fake)
    assert C.device_status(reset=False) == 105 and int(ws.count_nonzero()) == 4096   # reading alone changes nothing
    assert C.device_status(reset=True) == 105
    assert int(ws.count_nonzero()) == 0
    monkeypatch.undo()
    assert C.device_status() == 0
    # and a small-M linear through the cleared scratch is right
    from oracle import w8a8 as O
    g = torch.Generator().manual_seed(1)
    x = torch.randint(-127, 128, (8, 4096), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (2048, 4096), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (2048,), generator=g, dtype=torch.int8)
    assert torch.equal(C.linear_a8_w8_b8_o8(x.cuda(), w.cuda(), b.cuda(), 2e-4, 0.01).cpu(),
                       O.linear_a8_w8_b8_o8(x, w, b, 2e-4, 0.01))
