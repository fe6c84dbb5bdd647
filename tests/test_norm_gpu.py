"""Parity of the LayerNorm-quantise, dequant-add-LayerNorm-quantise and softmax-quantise
kernels with the CPU oracle (which calls the same torch functions the reference calls)."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_fp32_close, assert_quant_close, randn
from oracle import w8a8 as O

pytestmark = pytest.mark.gpu


def affine(h, seed, scale):
    g = torch.Generator().manual_seed(seed)
    return (1.0 + 0.1 * torch.randn(h, generator=g)) * scale, 0.1 * torch.randn(h, generator=g) * scale


def test_layernorm_q_golden(cuda_ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "layernorm_q.npz"))  # reference LayerNormQ.forward outputs
    for i in range(int(z["n"])):
        q = cuda_ops.layernorm_q(torch.from_numpy(z[f"x{i}"]).cuda(), torch.from_numpy(z[f"gamma{i}"]).cuda(),
                                 torch.from_numpy(z[f"beta{i}"]).cuda(), float(z[f"eps{i}"]))
        assert_quant_close(q, torch.from_numpy(z[f"q{i}"]), 0.999, f"golden case {i}")


@pytest.mark.parametrize("shape", [(1, 1, 4), (2, 3, 8), (3, 7, 100), (2, 5, 1026), (4, 512, 5120), (2, 64, 7168),
                                   (1, 32, 12288), (1, 3, 20480)])
def test_layernorm_q_vs_oracle(cuda_ops, shape):
    from torch_int.nn.fused import LayerNormQ
    h = shape[-1]
    x = randn(shape, 1, 2.0) + 0.3
    gamma, beta = affine(h, 2, 25.0)
    m = LayerNormQ(h)
    m.weight, m.bias = gamma, beta
    m = m.cuda()
    assert_quant_close(m(x.cuda()), O.layernorm_q(x, gamma, beta, 1e-5), 0.999, str(shape))
    assert_quant_close(m(x.half().cuda()), O.layernorm_q(x.half(), gamma, beta, 1e-5), 0.999, str(shape) + " fp16 in")


def test_dq_add_layernorm_q_golden(cuda_ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "dq_add_layernorm_q.npz"))  # reference dq_add_layernorm_q_py outputs
    for i in range(int(z["n"])):
        r, q = cuda_ops.dq_add_layernorm_q(torch.from_numpy(z[f"in{i}"]).cuda(), float(z[f"scale{i}"]),
                                           torch.from_numpy(z[f"res{i}"]).cuda(),
                                           torch.from_numpy(z[f"gamma{i}"]).cuda(),
                                           torch.from_numpy(z[f"beta{i}"]).cuda(), float(z[f"eps{i}"]))
        assert_fp32_close(r, torch.from_numpy(z[f"res_out{i}"]), 1e-5, f"residual, golden case {i}")
        assert_quant_close(q, torch.from_numpy(z[f"q{i}"]), 0.999, f"q, golden case {i}")


@pytest.mark.parametrize("shape", [(2, 3, 4), (1, 5, 90), (4, 512, 5120), (2, 128, 12288), (1, 2, 16388)])
def test_dq_add_layernorm_q_vs_oracle(cuda_ops, shape):
    h = shape[-1]
    g = torch.Generator().manual_seed(3)
    x = torch.randint(-200000, 200000, shape, generator=g, dtype=torch.int32)
    res = randn(shape, 4)
    gamma, beta = affine(h, 5, 30.0)
    scale = 1.3e-5
    r, q = cuda_ops.dq_add_layernorm_q(x.cuda(), scale, res.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
    r_o, q_o = O.dq_add_layernorm_q(x, scale, res, gamma, beta, 1e-5)
    assert torch.equal(r.cpu(), r_o), "residual output must be bit-exact (one fused multiply-add)"
    assert_quant_close(q, q_o, 0.999, str(shape))
    # the input tensors are not modified (fused.cu:17 uses an out-of-place add)
    assert torch.equal(res, randn(shape, 4))
    bias = randn((h,), 6, 0.5)
    r, q = cuda_ops.dq_add_layernorm_q_bias(x.cuda(), scale, bias.cuda(), res.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
    r_o, q_o = O.dq_add_layernorm_q_bias(x, scale, bias, res, gamma, beta, 1e-5)
    assert_fp32_close(r, r_o, 1e-6, "residual with bias")
    assert_quant_close(q, q_o, 0.999, str(shape) + " with bias")


def test_dq_add_layernorm_q_vs_reference_cpp(cuda_ops):
    """The GPU kernel against the reference's own C++ op (torch_int/kernels/fused.cu) compiled into
    oracle/_ref and run on CPU tensors; skipped where that module has not been built."""
    from oracle import build_ref
    ref = build_ref.load()
    if ref is None:
        pytest.skip("oracle/_ref/ref_fused.so is not built")
    for shape, scale in (((2, 3, 4), 0.01), ((4, 128, 5120), 1.3e-5), ((1, 64, 12288), 2e-5)):
        h = shape[-1]
        g = torch.Generator().manual_seed(h)
        x = torch.randint(-200000, 200000, shape, generator=g, dtype=torch.int32)
        res = randn(shape, 11)
        gamma, beta = affine(h, 12, 30.0)
        r_ref, q_ref = ref.dq_add_layernorm_q(x, scale, res, gamma, beta, 1e-5)
        r, q = cuda_ops.dq_add_layernorm_q(x.cuda(), scale, res.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
        assert torch.equal(r.cpu(), r_ref), f"residual output {shape}"
        assert_quant_close(q, q_ref, 0.999, f"q {shape}")


def test_fp16_residual_paths(cuda_ops):
    """The fp16 forms.  (1) dq_add_layernorm_q on an fp16 residual against the reference's own C++ op run on
    fp16 CPU tensors (its torch::add converts the int32 input to fp16, its layer_norm returns fp16): residual
    bit for bit, int8 within one unit at ties.  (2) The model's residual update with the linear folded in
    (fp32 linear output cast to fp16, added in fp16, LayerNormQ in fp32) against the oracle.  (3) LayerNormQ
    on an fp16 tensor with fp32 parameters (normalised in fp32) and with fp16 parameters."""
    from oracle import build_ref
    C = cuda_ops
    shape, h = (3, 40, 5120), 5120
    g = torch.Generator().manual_seed(31)
    x = torch.randint(-30000, 30000, shape, generator=g, dtype=torch.int32)      # within fp16 range, as the op needs
    res = randn(shape, 32).half()
    gamma, beta = affine(h, 33, 30.0)
    ref = build_ref.load()
    if ref is not None:
        # the reference's op is plain ATen code, so the same binary runs on CUDA tensors: there its
        # torch::add / layer_norm are ATen's CUDA kernels, i.e. the arithmetic the reference itself gets
        # (ATen's CUDA layer_norm wants parameters of the input's dtype: fp16 here; its CPU kernel takes fp32 ones)
        r_ref, q_ref = ref.dq_add_layernorm_q(x.cuda(), 2e-4, res.cuda(), gamma.cuda().half(), beta.cuda().half(), 1e-5)
        r, q = C.dq_add_layernorm_q(x.cuda(), 2e-4, res.cuda(), gamma.cuda().half().float(), beta.cuda().half().float(), 1e-5)
        assert r.dtype == torch.float16 and torch.equal(r, r_ref), "fp16 residual output vs the reference op on the GPU"
        assert_quant_close(q, q_ref, 0.995, "fp16 dq_add_layernorm_q vs the reference's C++ op")
        # on CPU tensors ATen rounds differently (the residual may differ by one fp16 unit)
        r_cpu, _ = ref.dq_add_layernorm_q(x, 2e-4, res, gamma, beta, 1e-5)
        assert torch.allclose(r.cpu().float(), r_cpu.float(), rtol=2e-3, atol=1e-3)
    big = torch.randint(-2000000, 2000000, shape, generator=g, dtype=torch.int32)  # accumulator-sized values
    bias = randn((h,), 34, 0.5)
    r, q = C.dq_add_layernorm_q_bias(big.cuda(), 3e-6, bias.cuda(), res.cuda(), gamma.cuda(), beta.cuda(), 1e-5)
    r_o, q_o = O.dq_add_layernorm_q_bias(big, 3e-6, bias, res, gamma, beta, 1e-5)
    assert r.dtype == torch.float16 and torch.equal(r.cpu(), r_o), "model residual update in fp16"
    assert_quant_close(q, q_o, 0.999, "LayerNormQ after the fp16 residual update")
    xh = randn(shape, 35, 3.0).half()
    assert_quant_close(C.layernorm_q(xh.cuda(), gamma.cuda(), beta.cuda(), 1e-5), O.layernorm_q(xh, gamma, beta, 1e-5),
                       0.999, "fp16 input, fp32 LayerNorm")
    assert_quant_close(C.layernorm_q(xh.cuda(), gamma.cuda(), beta.cuda(), 1e-5, fp32_norm=False),
                       O.layernorm_q(xh, gamma.half(), beta.half(), 1e-5), 0.995, "fp16 input and parameters")


def test_dq_add_module(cuda_ops):
    from torch_int.nn.fused import DQ_Add_LayerNorm_Q
    m = DQ_Add_LayerNorm_Q(256).cuda()
    m.input_scale = 0.002
    g = torch.Generator().manual_seed(7)
    x = torch.randint(-65536, 65536, (2, 9, 256), generator=g, dtype=torch.int32)
    res = randn((2, 9, 256), 8)
    r, q = m(res.cuda(), x.cuda())
    r_o, q_o = O.dq_add_layernorm_q(x, 0.002, res, torch.ones(256), torch.zeros(256), 1e-5)
    assert torch.equal(r.cpu(), r_o)
    assert_quant_close(q, q_o, 0.999)


@pytest.mark.parametrize("bsz,heads,t,s", [(1, 1, 1, 16), (2, 3, 16, 16), (2, 4, 48, 112), (1, 5, 512, 512),
                                           (1, 2, 16, 2048), (2, 2, 1, 528), (1, 1, 3, 2064), (1, 3, 40, 1040)])
def test_softmax_q(cuda_ops, bsz, heads, t, s):
    scores = randn((bsz * heads, t, s), 9, 2.5)
    mask = O.causal_mask(bsz, t, s)
    want = O.softmax_q(scores, mask)
    assert_quant_close(cuda_ops.softmax_q(scores.cuda(), mask.cuda(), heads), want, 0.999, "explicit mask")
    assert_quant_close(cuda_ops.softmax_q(scores.cuda(), None, heads, causal=s - t), want, 0.999, "generated mask")
    assert_quant_close(cuda_ops.softmax_q(scores.cuda()), O.softmax_q(scores), 0.999, "no mask")
    # padding mask: a fully masked key column range
    pad = mask.clone()
    pad[:, :, :, : s // 4] = torch.finfo(torch.float32).min
    assert_quant_close(cuda_ops.softmax_q(scores.cuda(), pad.cuda(), heads), O.softmax_q(scores, pad), 0.999, "padding")


@pytest.mark.parametrize("b,t,h,d,cap,col0", [(2, 48, 3, 128, 64, 16), (1, 1, 5, 64, 32, 7), (3, 130, 2, 128, 144, 0),
                                              (2, 512, 4, 128, 512, 0)])
def test_transpose_values(cuda_ops, b, t, h, d, cap, col0):
    g = torch.Generator().manual_seed(10)
    v = torch.randint(-128, 128, (b, t, h, d), generator=g, dtype=torch.int8)
    vt = torch.full((b, h, d, cap), 77, dtype=torch.int8, device="cuda")
    cuda_ops.transpose_values(v.cuda(), vt, col0)
    want = torch.full((b, h, d, cap), 77, dtype=torch.int8)
    want[..., col0:col0 + t] = v.permute(0, 2, 3, 1)   # value_states.transpose(1, 2) of opt.py:180
    assert torch.equal(vt.cpu(), want)
