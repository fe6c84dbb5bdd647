"""Parity of the three batched int8 products with the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_bit_exact, assert_fp32_close, rand_s8
from oracle import w8a8 as O

pytestmark = pytest.mark.gpu


def run_all(C, a, b, alpha, what):
    ac, bc = a.cuda(), b.cuda()
    assert_bit_exact(C.bmm_s8t_s8n_s32t(ac, bc), O.bmm_s8t_s8n_s32t(a, b), what + " s32t")
    assert_bit_exact(C.bmm_s8t_s8n_s8t(ac, bc, alpha), O.bmm_s8t_s8n_s8t(a, b, alpha), what + " s8t")
    assert_fp32_close(C.bmm_s8t_s8n_f32t(ac, bc, alpha), O.bmm_s8t_s8n_f32t(a, b, alpha), 1e-5, what + " f32t")


def test_reference_test_shapes(cuda_ops):
    # tests/test_bmm.py:9-11: B, M, K, N = 1, 512, 512, 32, scale 0.001
    a, b = rand_s8((1, 512, 512), 0, -128, 126), rand_s8((1, 32, 512), 1, -128, 126)
    run_all(cuda_ops, a, b, 0.001, "1x512x32x512")
    # tests/test_bmm.py:114: N = 12288, int32 out
    a, b = rand_s8((1, 512, 512), 2, -128, 126), rand_s8((1, 12288, 512), 3, -128, 126)
    assert_bit_exact(cuda_ops.bmm_s8t_s8n_s32t(a.cuda(), b.cuda()), O.bmm_s8t_s8n_s32t(a, b))


def test_known_answer_and_formulas(cuda_ops, golden_dir):
    C = cuda_ops
    z = np.load(os.path.join(golden_dir, "bmm_known_answer.npz"))  # tests/test_bmm.py:34-106
    a = torch.from_numpy(z["a"])
    b = torch.from_numpy(z["b_kn"]).transpose(1, 2).contiguous()
    c = C.bmm_s8t_s8n_s8t(a.cuda(), b.cuda(), float(z["scale"])).cpu()
    d = (c.int() - torch.from_numpy(z["c"]).int()).abs()
    assert int(d.max()) <= 1 and float((d == 0).double().mean()) >= 0.99
    assert_bit_exact(c, O.bmm_s8t_s8n_s8t(a, b, float(z["scale"])))
    z = np.load(os.path.join(golden_dir, "bmm_formulas.npz"))      # tests/test_bmm.py:7-30,112-120
    a, b, s = torch.from_numpy(z["a"]), torch.from_numpy(z["b"]), float(z["scale"])
    assert torch.equal(C.bmm_s8t_s8n_s32t(a.cuda(), b.cuda()).cpu(), torch.from_numpy(z["gt_s32"]))
    d = (C.bmm_s8t_s8n_s8t(a.cuda(), b.cuda(), s).cpu().int() - torch.from_numpy(z["gt_s8"]).int()).abs()
    assert int(d.max()) <= 1 and float((d == 0).double().mean()) >= 0.999
    mse = torch.mean((C.bmm_s8t_s8n_f32t(a.cuda(), b.cuda(), s).cpu() - torch.from_numpy(z["gt_f32"])) ** 2)
    assert float(mse) < 1e-8


def test_minimum_shapes(cuda_ops):
    # tests/test_bmm_shape.py:6-26
    a, b = rand_s8((1, 1, 16), 4), rand_s8((1, 4, 16), 5)
    assert_fp32_close(cuda_ops.bmm_s8t_s8n_f32t(a.cuda(), b.cuda(), 0.001), O.bmm_s8t_s8n_f32t(a, b, 0.001), 1e-5)
    b = rand_s8((1, 16, 16), 6)
    assert_bit_exact(cuda_ops.bmm_s8t_s8n_s8t(a.cuda(), b.cuda(), 0.001), O.bmm_s8t_s8n_s8t(a, b, 0.001))


@pytest.mark.parametrize("shape", [(3, 1, 16, 16), (5, 77, 48, 80), (2, 130, 272, 144), (7, 129, 16, 1040),
                                   (160, 16, 128, 528)])
def test_ragged(cuda_ops, shape):
    bsz, m, n, k = shape
    a, b = rand_s8((bsz, m, k), 7), rand_s8((bsz, n, k), 8)
    run_all(cuda_ops, a, b, 1.0 / (50.0 * k ** 0.5), str(shape))


@pytest.mark.parametrize("seq", [128, 512, 2048])
def test_attention_sweep(cuda_ops, seq):
    """batch*heads = 4*40, head_dim 128: Q.K^T with alpha = 1/127^2 (fp32 out) and P.V with
    alpha = 0.01 (int8 out), plus P.V at alpha ~ 1/sigma(acc) so that rounding is exercised."""
    C = cuda_ops
    bh, d = 160, 128
    q, k = rand_s8((bh, seq, d), 10), rand_s8((bh, seq, d), 11)
    assert_fp32_close(C.bmm_s8t_s8n_f32t(q.cuda(), k.cuda(), 1.0 / 127 ** 2),
                      O.bmm_s8t_s8n_f32t(q, k, 1.0 / 127 ** 2), 1e-5, f"QK^T S={seq}")
    p, vt = rand_s8((bh, seq, seq), 12), rand_s8((bh, d, seq), 13)
    assert_bit_exact(C.bmm_s8t_s8n_s8t(p.cuda(), vt.cuda(), 0.01), O.bmm_s8t_s8n_s8t(p, vt, 0.01), f"PV S={seq}")
    alpha = 1.0 / (73.0 * 73.0 * seq ** 0.5) * 40
    assert_bit_exact(C.bmm_s8t_s8n_s8t(p.cuda(), vt.cuda(), alpha), O.bmm_s8t_s8n_s8t(p, vt, alpha),
                     f"PV S={seq} unsaturated")
    assert C.device_status() == 0


def test_strided_views_without_copies(cuda_ops):
    """ti_gemm_i8_ex on [B,T,H,D] projections addressed as (b,h) batches: equals the packed
    product on transposed contiguous copies (what torch_int/models/opt.py:80-81 makes)."""
    C = cuda_ops
    bsz, t, h, d = 2, 48, 3, 128
    e = h * d
    q, k = rand_s8((bsz, t, e), 14), rand_s8((bsz, t, e), 15)
    out = torch.empty((bsz * h, t, t), dtype=torch.float32, device="cuda")
    C.gemm_i8_ex(q.cuda(), k.cuda(), out, epilogue=C.EPI_F32_ALPHA, m=t, n=t, k=d, batch=h, batch2=bsz,
                 lda=e, ldb=e, ldc=t, stride_a=d, stride_b=d, stride_c=t * t,
                 stride2_a=t * e, stride2_b=t * e, stride2_c=h * t * t, alpha=0.01)
    qh = q.view(bsz, t, h, d).transpose(1, 2).reshape(bsz * h, t, d).contiguous()
    kh = k.view(bsz, t, h, d).transpose(1, 2).reshape(bsz * h, t, d).contiguous()
    assert_fp32_close(out, O.bmm_s8t_s8n_f32t(qh, kh, 0.01), 1e-5, "strided QK^T")


def test_rejects_bad_arguments(cuda_ops):
    C = cuda_ops
    a, b = rand_s8((2, 4, 32), 1).cuda(), rand_s8((2, 16, 32), 2).cuda()
    with pytest.raises(RuntimeError):
        C.bmm_s8t_s8n_s8t(a, b[:1], 1.0)
    with pytest.raises(RuntimeError):
        C.bmm_s8t_s8n_s8t(a, rand_s8((2, 16, 48), 2).cuda(), 1.0)
    with pytest.raises(RuntimeError, match="N=20"):
        C.bmm_s8t_s8n_s8t(a, rand_s8((2, 20, 32), 2).cuda(), 1.0)
    assert C.bmm_s8t_s8n_s32t(a[:0], b[:0]).shape == (0, 4, 16)
