"""Cross-checks inside the oracle: the C restatement against its numpy twin and
against float64 BLAS, and the host's torch.add against a fused multiply-add.  No GPU."""
import numpy as np
import pytest
import torch

from helpers import rand_s8, rand_s32, randn
from oracle import w8a8 as O


@pytest.mark.parametrize("shape", [(1, 16, 16), (3, 20, 48), (37, 52, 80), (64, 96, 256), (5, 7, 1040)])
def test_contraction_c_vs_numpy_vs_fp64(shape):
    m, n, k = shape
    a, b = rand_s8((m, k), 1, -128, 127), rand_s8((n, k), 2, -128, 127)
    acc = O.gemm_acc(a, b)
    assert torch.equal(acc, O.gemm_acc(a, b, naive=True))
    assert torch.equal(acc, O.gemm_acc_numpy(a, b))
    assert torch.equal(acc, O.gemm_acc_fp64(a, b))


def test_contraction_batched_and_extremes():
    a = torch.full((2, 9, 512), -128, dtype=torch.int8)
    b = torch.full((2, 5, 512), -128, dtype=torch.int8)
    assert int(O.gemm_acc(a, b).max()) == 512 * 128 * 128
    a, b = rand_s8((4, 33, 64), 3), rand_s8((4, 17, 64), 4)
    assert torch.equal(O.gemm_acc(a, b), O.gemm_acc_numpy(a, b))
    assert O.gemm_acc(torch.empty((0, 16), dtype=torch.int8), torch.empty((4, 16), dtype=torch.int8)).shape == (0, 4)


def test_large_contraction_c_vs_fp64():
    a, b = rand_s8((256, 4096), 5), rand_s8((384, 4096), 6)
    assert torch.equal(O.gemm_acc(a, b), O.gemm_acc_fp64(a, b))


@pytest.mark.parametrize("alpha,beta", [(0.001, 0.01), (1e-4, 0.01), (0.37, 1.0), (3.0, 100.0)])
def test_epilogues_c_vs_numpy(alpha, beta):
    x, w = rand_s8((40, 128), 7), rand_s8((48, 128), 8)
    b8, b32, bf = rand_s8((48,), 9), rand_s32((48,), 10), randn((48,), 11)
    acc = O.gemm_acc(x, w)
    pairs = [
        (O.linear_a8_w8_b8_o8(x, w, b8, alpha, beta), O.epilogue_numpy(acc, b8, alpha, beta, "b8_o8")),
        (O.linear_relu_a8_w8_b8_o8(x, w, b8, alpha, beta), O.epilogue_numpy(acc, b8, alpha, beta, "relu_b8_o8")),
        (O.linear_a8_w8_b32_o32_with_scaling(x, w, b32, alpha, beta * 1e-6),
         O.epilogue_numpy(acc, b32, alpha, beta * 1e-6, "b32_o32_with_scaling")),
        (O.linear_a8_w8_b32_o32(x, w, b32), O.epilogue_numpy(acc, b32, 1, 1, "b32_o32")),
        (O.bmm_s8t_s8n_s8t(x[None], w[None], alpha)[0], O.epilogue_numpy(acc, None, alpha, 0, "s8t")),
        (O.bmm_s8t_s8n_s32t(x[None], w[None])[0], O.epilogue_numpy(acc, None, 1, 0, "s32t")),
    ]
    for i, (c_out, np_out) in enumerate(pairs):
        assert torch.equal(c_out, np_out), f"pair {i}"
    # fp32 outputs: the float64-emulated FMA may differ from a true FMA by one ulp in
    # rare double-rounding cases; everything else must be identical.
    for c_out, np_out in [
        (O.linear_a8_w8_bfp32_ofp32(x, w, bf, alpha, beta), O.epilogue_numpy(acc, bf, alpha, beta, "bfp32_ofp32")),
        (O.bmm_s8t_s8n_f32t(x[None], w[None], alpha)[0], O.epilogue_numpy(acc, None, alpha, 0, "f32t")),
    ]:
        assert float((c_out != np_out).double().mean()) < 1e-3
        assert torch.allclose(c_out, np_out, rtol=2e-7, atol=0)


def test_saturation_and_ties():
    # acc values chosen so that alpha*acc lands exactly on .5 ties and far outside int8.
    x = torch.tensor([[1, 0], [3, 0], [5, 0], [-1, 0], [-3, 0], [127, 127], [-128, -128]], dtype=torch.int8)
    x = torch.cat([x, torch.zeros((7, 14), dtype=torch.int8)], dim=1)
    w = torch.zeros((16, 16), dtype=torch.int8)
    w[:, 0] = 1
    w[:, 1] = 127
    zero = torch.zeros(16, dtype=torch.int8)
    y = O.linear_a8_w8_b8_o8(x, w, zero, 0.5, 0.0)
    assert y[:, 0].tolist() == [0, 2, 2, 0, -2, 127, -128]  # half to even, then saturation
    y = O.linear_relu_a8_w8_b8_o8(x, w, zero, 0.5, 0.0)
    assert y[:, 0].tolist() == [0, 2, 2, 0, 0, 127, 0]


def test_host_torch_add_is_fused():
    """dq_add_layernorm_q's first step is torch.add(residual, int32, alpha): the
    kernel implements it as fma(scale, f32(in), residual).  Check what this
    host's torch does, so a mismatch in the GPU parity test can be attributed."""
    g = torch.Generator().manual_seed(0)
    inp = torch.randint(-65536, 65536, (4096,), generator=g, dtype=torch.int32)
    res = torch.randn(4096, generator=g)
    scale = 0.01
    got = torch.add(res, inp, alpha=scale).numpy()
    fused = (np.float64(np.float32(scale)) * inp.numpy().astype(np.float32).astype(np.float64)
             + res.numpy().astype(np.float64)).astype(np.float32)
    unfused = (np.float32(scale) * inp.numpy().astype(np.float32)).astype(np.float32) + res.numpy()
    n_fused, n_unfused = int((got != fused).sum()), int((got != unfused).sum())
    assert min(n_fused, n_unfused) == 0, (n_fused, n_unfused)


def test_softmax_q_and_mask():
    s = randn((6, 5, 16), 12, 3.0)
    mask = O.causal_mask(2, 5, 16)
    p = O.softmax_q(s, mask)
    assert p.dtype == torch.int8 and int(p.min()) >= 0 and int(p.max()) <= 127
    # masked (future) positions are exactly zero; rows sum to about 127
    assert int(p[:, 0, 12:].abs().sum()) == 0
    assert (p.int().sum(-1) - 127).abs().max() <= 8
