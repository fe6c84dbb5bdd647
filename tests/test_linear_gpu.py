"""Parity of the five W8A8 linear ops (through the C ABI) with the CPU oracle.
int32 and int8 outputs must be bit-exact, fp32 outputs within 1e-5 relative."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_bit_exact, assert_fp32_close, rand_s8, rand_s32, randn
from oracle import w8a8 as O

pytestmark = pytest.mark.gpu


def run_all(C, x, w, b8, b32, bf, alpha, beta, what):
    xc, wc = x.cuda(), w.cuda()
    assert_bit_exact(C.linear_a8_w8_b32_o32(xc, wc, b32.cuda()), O.linear_a8_w8_b32_o32(x, w, b32), what + " b32_o32")
    assert_bit_exact(C.linear_a8_w8_b8_o8(xc, wc, b8.cuda(), alpha, beta),
                     O.linear_a8_w8_b8_o8(x, w, b8, alpha, beta), what + " b8_o8")
    assert_bit_exact(C.linear_relu_a8_w8_b8_o8(xc, wc, b8.cuda(), alpha, beta),
                     O.linear_relu_a8_w8_b8_o8(x, w, b8, alpha, beta), what + " relu_b8_o8")
    assert_bit_exact(C.linear_a8_w8_b32_o32_with_scaling(xc, wc, b32.cuda(), alpha, beta * 1e-7),
                     O.linear_a8_w8_b32_o32_with_scaling(x, w, b32, alpha, beta * 1e-7), what + " b32_o32_scaling")
    assert_fp32_close(C.linear_a8_w8_bfp32_ofp32(xc, wc, bf.cuda(), alpha, 1.0),
                      O.linear_a8_w8_bfp32_ofp32(x, w, bf, alpha, 1.0), 1e-5, what + " bfp32_ofp32")


def test_reference_test_shapes(cuda_ops):
    # rows 128, K 512, N 1024, inputs randint(-128, 127) as tests/test_linear_kernels.py:8-12
    x, w = rand_s8((128, 512), 0, -128, 126), rand_s8((1024, 512), 1, -128, 126)
    b8, b32, bf = rand_s8((1024,), 2, -128, 126), rand_s32((1024,), 3), randn((1024,), 4)
    run_all(cuda_ops, x, w, b8, b32, bf, 0.001, 0.01, "128x1024x512")
    assert cuda_ops.device_status() == 0


def test_reference_formulas_with_their_tolerances(cuda_ops, golden_dir):
    # The ground truths of tests/test_linear_kernels.py, evaluated by that file's own
    # formulas when the fixture was generated, with that file's tolerances.
    z = np.load(os.path.join(golden_dir, "linear_formulas.npz"))
    C = cuda_ops
    x, w = torch.from_numpy(z["x"]).cuda(), torch.from_numpy(z["w"]).cuda()
    b32, b8, bf = (torch.from_numpy(z[k]).cuda() for k in ("b32", "b8", "bf"))
    ab, atol = z["alpha_beta"], z["atol"]
    y = C.linear_a8_w8_b32_o32_with_scaling(x, w, b32, *ab[1]).cpu()
    assert torch.allclose(torch.from_numpy(z["gt_b32_o32_scaling"]), y.float(), atol=float(atol[1]), rtol=1e-6)
    y = C.linear_a8_w8_bfp32_ofp32(x, w, bf, *ab[2]).cpu()
    assert torch.allclose(torch.from_numpy(z["gt_bfp32_ofp32"]), y, atol=float(atol[2]))
    y = C.linear_a8_w8_b8_o8(x, w, b8, *ab[3]).cpu()
    assert torch.allclose(torch.from_numpy(z["gt_b8_o8"]), y.float(), atol=float(atol[3]))
    y = C.linear_relu_a8_w8_b8_o8(x, w, b8, *ab[4]).cpu()
    assert torch.allclose(torch.from_numpy(z["gt_relu_b8_o8"]), y.float(), atol=float(atol[4]))


def test_minimum_shapes(cuda_ops):
    # tests/test_linear_shape.py:8-37: rows 1, K 16, N 4 (fp32 out) and N 16 (int8 out)
    C = cuda_ops
    x, w = rand_s8((1, 16), 5), rand_s8((4, 16), 6)
    bf = randn((4,), 7)
    assert_fp32_close(C.linear_a8_w8_bfp32_ofp32(x.cuda(), w.cuda(), bf.cuda(), 0.001, 1.0),
                      O.linear_a8_w8_bfp32_ofp32(x, w, bf, 0.001, 1.0), 1e-5, "1x4x16")
    b32 = rand_s32((4,), 8)
    assert_bit_exact(C.linear_a8_w8_b32_o32(x.cuda(), w.cuda(), b32.cuda()), O.linear_a8_w8_b32_o32(x, w, b32))
    w, b8 = rand_s8((16, 16), 9), rand_s8((16,), 10)
    assert_bit_exact(C.linear_a8_w8_b8_o8(x.cuda(), w.cuda(), b8.cuda(), 0.001, 0.01),
                     O.linear_a8_w8_b8_o8(x, w, b8, 0.001, 0.01))


@pytest.mark.parametrize("m,n,k", [(1, 16, 16), (7, 48, 80), (127, 272, 144), (129, 240, 1040), (300, 528, 400),
                                   (2, 1040, 2064), (513, 16, 4096), (8, 7168, 512), (16, 96, 12288)])
def test_ragged_tiles(cuda_ops, m, n, k):
    """M, N and K tails relative to the 128 x BN x 128 tiles, every N tile width."""
    x, w = rand_s8((m, k), m + n), rand_s8((n, k), k)
    b8, b32, bf = rand_s8((n,), 1), rand_s32((n,), 2), randn((n,), 3)
    run_all(cuda_ops, x, w, b8, b32, bf, 1.0 / (60.0 * k ** 0.5), 0.01, f"{m}x{n}x{k}")


@pytest.mark.parametrize("tile_n,cta_pair", [(32, 1), (64, 1), (128, 1), (256, 1), (256, 2)])
def test_every_tile_shape(cuda_ops, tile_n, cta_pair):
    """Every N tile width of the single-CTA kernel and the 256 x 256 CTA-pair kernel."""
    C = cuda_ops
    m, n, k = 600, 400, 272
    x, w, b8 = rand_s8((m, k), 20), rand_s8((n, k), 21), rand_s8((n,), 22)
    out = torch.empty((m, n), dtype=torch.int8, device="cuda")
    C.gemm_i8_ex(x.cuda(), w.cuda(), out, b8.cuda(), epilogue=C.EPI_S8_BIAS_S8, m=m, n=n, k=k,
                 lda=k, ldb=k, ldc=n, alpha=0.002, beta=0.05, tile_n=tile_n, cta_pair=cta_pair)
    assert_bit_exact(out, O.linear_a8_w8_b8_o8(x, w, b8, 0.002, 0.05), f"tile_n={tile_n} cta_pair={cta_pair}")
    bf = randn((n,), 23)
    outf = torch.empty((m, n), dtype=torch.float32, device="cuda")
    C.gemm_i8_ex(x.cuda(), w.cuda(), outf, bf.cuda(), epilogue=C.EPI_F32_BIAS_F32, m=m, n=n, k=k,
                 lda=k, ldb=k, ldc=n, alpha=0.002, beta=1.0, tile_n=tile_n, cta_pair=cta_pair)
    assert_fp32_close(outf, O.linear_a8_w8_bfp32_ofp32(x, w, bf, 0.002, 1.0), 1e-5, f"fp32 tile_n={tile_n}")
    assert C.device_status() == 0


def test_config_single_linear(cuda_ops):
    """x [4,128,4096], W [4096,4096], bias [4096] uniform on [-127,127], alpha=0.001, beta=0.01,
    seed 0; plus the same inputs with alpha=1e-4 so that most outputs do not saturate."""
    from torch_int.nn.linear import W8A8B8O8Linear
    g = torch.Generator().manual_seed(0)
    x = torch.randint(-127, 128, (4, 128, 4096), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (4096, 4096), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (4096,), generator=g, dtype=torch.int8)
    for alpha in (0.001, 1e-4):
        m = W8A8B8O8Linear(4096, 4096, alpha=alpha, beta=0.01)
        m.weight, m.bias = w, b.view(1, -1)
        m = m.to("cuda")
        y = m(x.cuda())
        assert y.shape == (4, 128, 4096) and y.dtype == torch.int8
        want = O.linear_a8_w8_b8_o8(x.view(-1, 4096), w, b, alpha, 0.01).view(4, 128, 4096)
        assert_bit_exact(y, want, f"config 1, alpha={alpha}")
    sat = float(((want == 127) | (want == -128)).double().mean())
    assert sat < 0.2, "the alpha=1e-4 run must exercise the rounding path"


def test_headline_gemm_full_tensor(cuda_ops):
    """4096 x 12288 x 12288, int8 out, alpha=1e-4, beta=0.01: every element against the oracle."""
    C = cuda_ops
    x, w, b8 = rand_s8((4096, 12288), 100), rand_s8((12288, 12288), 101), rand_s8((12288,), 102)
    y = C.linear_a8_w8_b8_o8(x.cuda(), w.cuda(), b8.cuda(), 1e-4, 0.01)
    assert_bit_exact(y, O.linear_a8_w8_b8_o8(x, w, b8, 1e-4, 0.01), "headline GEMM")
    assert cuda_ops.device_status() == 0


@pytest.mark.parametrize("m,n,k,what", [
    (4096, 7168, 7168, "OPT-30B q/k/v/out_proj, batch 8 x 512"),
    (4096, 28672, 7168, "OPT-30B fc1"),
    (4096, 7168, 28672, "OPT-30B fc2"),
    (16384, 12288, 1536, "OPT-175B out_proj shard of one of 8 ranks, batch 16 x 1024"),
    (16, 9216, 12288, "OPT-175B q/k/v shard of one of 4 ranks, decode step"),
    (16, 12288, 3072, "OPT-175B out_proj shard of one of 4 ranks, decode step"),
])
def test_model_layer_shapes_full_tensor(cuda_ops, m, n, k, what):
    """The GEMMs of the benchmarked models at their full per-layer (and per-rank) shapes, every element
    against the oracle, in the epilogue the model uses there: int8 out with bias for the column-parallel
    projections, raw int32 partial sums for the row-parallel ones."""
    C = cuda_ops
    x, w = rand_s8((m, k), 200 + m % 7), rand_s8((n, k), 201 + n % 7)
    acc = torch.empty((m, n), dtype=torch.int32, device="cuda")
    C.gemm_i8_ex(x.cuda(), w.cuda(), acc, epilogue=C.EPI_S32_RAW, m=m, n=n, k=k, lda=k, ldb=k, ldc=n)
    want = O.gemm_acc(x, w)
    assert_bit_exact(acc, want, what + " (int32 partial sums)")
    del acc
    b8 = rand_s8((n,), 202)
    alpha = 1.0 / (60.0 * k ** 0.5)
    y = C.linear_relu_a8_w8_b8_o8(x.cuda(), w.cuda(), b8.cuda(), alpha, 0.05)
    assert_bit_exact(y, O.epilogue_s8_bias_s8(want, b8, alpha, 0.05, relu=True), what + " (ReLU int8)")
    ws = C._split_k_workspace(torch.device("cuda", torch.cuda.current_device()))
    assert int(ws.count_nonzero()) == 0, "the scratch of the split paths must be left zeroed"
    assert C.device_status() == 0


def test_linearity_property_at_full_size(cuda_ops):
    """Size-independent property: with int32 outputs, (x1 + x2) W^T == x1 W^T + x2 W^T."""
    C = cuda_ops
    m, n, k = 2048, 5120, 20480
    x1, x2 = rand_s8((m, k), 30, -63, 63).cuda(), rand_s8((m, k), 31, -63, 63).cuda()
    w = rand_s8((n, k), 32).cuda()
    zero = torch.zeros(n, dtype=torch.int32, device="cuda")
    y12 = C.linear_a8_w8_b32_o32((x1 + x2), w, zero)
    y1, y2 = C.linear_a8_w8_b32_o32(x1, w, zero), C.linear_a8_w8_b32_o32(x2, w, zero)
    assert torch.equal(y12, y1 + y2)


def test_rejects_bad_arguments(cuda_ops):
    C = cuda_ops
    x, w = rand_s8((4, 32), 1).cuda(), rand_s8((16, 32), 2).cuda()
    b = rand_s8((16,), 3).cuda()
    with pytest.raises(RuntimeError, match="dtype"):
        C.linear_a8_w8_b8_o8(x.float(), w, b, 1.0, 1.0)
    with pytest.raises(RuntimeError, match="contiguous"):
        C.linear_a8_w8_b8_o8(rand_s8((32, 4), 1).cuda().t(), w, b, 1.0, 1.0)
    with pytest.raises(RuntimeError, match="disagree"):
        C.linear_a8_w8_b8_o8(x, rand_s8((16, 48), 2).cuda(), b, 1.0, 1.0)
    with pytest.raises(RuntimeError, match="elements"):
        C.linear_a8_w8_b8_o8(x, w, b[:8], 1.0, 1.0)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        C.linear_a8_w8_b8_o8(rand_s8((4, 24), 1).cuda(), rand_s8((16, 24), 2).cuda(), b, 1.0, 1.0)
    # bias of any shape with N elements, on any device (linear.cu:420)
    y = C.linear_a8_w8_b8_o8(x, w, b.cpu().view(1, 16), 0.01, 0.1)
    assert_bit_exact(y, O.linear_a8_w8_b8_o8(x.cpu(), w.cpu(), b.cpu(), 0.01, 0.1))
    # empty batch
    assert C.linear_a8_w8_b8_o8(x[:0], w, b, 1.0, 1.0).shape == (0, 16)


@pytest.mark.parametrize("m,n,k", [(1, 7168, 7168), (8, 21504, 7168), (16, 1040, 28672), (128, 4096, 4096), (3, 48, 2048),
                                   (8, 50272, 2048), (5, 4112, 2064)])
def test_split_k_small_m(cuda_ops, m, n, k):
    """Few rows, long K (decode steps): K is split over the SMs, partial sums meet in a scratch
    workspace, the last CTA of a tile applies the epilogue.  Results must not change, twice in a row
    (the workspace has to come back zeroed)."""
    C = cuda_ops
    x, w = rand_s8((m, k), 41), rand_s8((n, k), 42)
    b8, b32, bf = rand_s8((n,), 43), rand_s32((n,), 44), randn((n,), 45)
    alpha = 1.0 / (60.0 * k ** 0.5)
    for _ in range(2):
        run_all(C, x, w, b8, b32, bf, alpha, 0.01, f"split-K {m}x{n}x{k}")
    C.set_narrow_a(0)  # the 128-row A stages that problems of more than 16 rows use
    try:
        out = torch.empty((m, n), dtype=torch.int8, device="cuda")
        C.gemm_i8_ex(x.cuda(), w.cuda(), out, b8.cuda(), epilogue=C.EPI_S8_BIAS_S8, m=m, n=n, k=k,
                     lda=k, ldb=k, ldc=n, alpha=alpha, beta=0.01)
    finally:
        C.set_narrow_a(1)
    assert_bit_exact(out, O.linear_a8_w8_b8_o8(x, w, b8, alpha, 0.01), "128-row A stages")
    for tile_n in (64, 128, 256):  # 64 has no narrow form
        out = torch.empty((m, n), dtype=torch.int8, device="cuda")
        C.gemm_i8_ex(x.cuda(), w.cuda(), out, b8.cuda(), epilogue=C.EPI_S8_BIAS_S8, m=m, n=n, k=k,
                     lda=k, ldb=k, ldc=n, alpha=alpha, beta=0.01, tile_n=tile_n, cta_pair=1)
        assert_bit_exact(out, O.linear_a8_w8_b8_o8(x, w, b8, alpha, 0.01), f"tile_n={tile_n}")
    for splits in (1, 2, 5, 16):
        out = torch.empty((m, n), dtype=torch.int8, device="cuda")
        C.gemm_i8_ex(x.cuda(), w.cuda(), out, b8.cuda(), epilogue=C.EPI_S8_BIAS_S8, m=m, n=n, k=k,
                     lda=k, ldb=k, ldc=n, alpha=alpha, beta=0.01, splits=splits)
        assert_bit_exact(out, O.linear_a8_w8_b8_o8(x, w, b8, alpha, 0.01), f"splits={splits}")
    ws = C._split_k_workspace(torch.device("cuda", torch.cuda.current_device()))
    assert int(ws.count_nonzero()) == 0, "the split-K workspace must be left zeroed"
    assert C.device_status() == 0


@pytest.mark.parametrize("m,n,k", [(4096, 7168, 7168), (300, 1040, 528), (130, 48, 2048), (8, 7168, 7168), (1, 16, 16)])
def test_fp32_epilogue_that_adds_to_c(cuda_ops, m, n, k):
    """C += fma(alpha, acc, bias): the fp32-output linear with the residual add of the decoder layer folded into
    its epilogue.  The sum must be exactly fp32(C + y) with y the value the plain fp32 epilogue stores."""
    C = cuda_ops
    x, w, bf = rand_s8((m, k), 61), rand_s8((n, k), 62), randn((n,), 63)
    alpha = 1.0 / (60.0 * k ** 0.5)
    start = randn((m, n), 64)
    y = C.linear_a8_w8_bfp32_ofp32(x.cuda(), w.cuda(), bf.cuda(), alpha, 1.0)
    assert_fp32_close(y, O.linear_a8_w8_bfp32_ofp32(x, w, bf, alpha, 1.0), 1e-5, "plain fp32 epilogue")
    out = start.cuda()
    C.gemm_i8_ex(x.cuda(), w.cuda(), out, bf.cuda(), epilogue=C.EPI_F32_BIAS_F32_ACC, m=m, n=n, k=k, lda=k, ldb=k,
                 ldc=n, alpha=alpha, beta=1.0)
    assert_bit_exact((start.cuda() + y).view(torch.int32), out.view(torch.int32), f"C += y at {m}x{n}x{k}")
    wide = torch.full((m, n + 16), 7.0, device="cuda")   # a view into a wider tensor: the columns beyond N stay
    wide[:, :n] = start.cuda()
    C.gemm_i8_ex(x.cuda(), w.cuda(), wide, bf.cuda(), epilogue=C.EPI_F32_BIAS_F32_ACC, m=m, n=n, k=k, lda=k, ldb=k,
                 ldc=n + 16, alpha=alpha, beta=1.0)
    assert_bit_exact(wide[:, :n].contiguous().view(torch.int32), out.view(torch.int32), "strided C")
    assert bool((wide[:, n:] == 7.0).all())
    assert C.device_status() == 0
