"""The REFERENCE's own CUDA kernels, built from its sources (oracle/build_ref_gemm.py -> oracle/_ref/
ref_torch_int.so, CUTLASS 2.x Sm80 mma.sync code translated by the driver for this GPU), run side by side
with this library on the same seeded inputs.  This is the run of the reference itself that pins the last bit
of the float GEMM epilogues, which the oracle can only restate.  Skipped where the module is not built."""
import pytest
import torch

from helpers import assert_bit_exact, assert_fp32_close, rand_s8, rand_s32, randn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref_gemm
    mod = build_ref_gemm.load()
    if mod is None:
        pytest.skip("oracle/_ref/ref_torch_int.so is not built (python oracle/build_ref_gemm.py)")
    return mod


def test_config_single_linear_vs_reference_kernel(cuda_ops, ref):
    """BASELINE config 1: x [4,128,4096], W [4096,4096], bias [4096], alpha = 0.001 (and 1e-4), beta = 0.01."""
    g = torch.Generator().manual_seed(0)
    x = torch.randint(-127, 128, (512, 4096), generator=g, dtype=torch.int8).cuda()
    w = torch.randint(-127, 128, (4096, 4096), generator=g, dtype=torch.int8).cuda()
    b = torch.randint(-127, 128, (4096,), generator=g, dtype=torch.int8).cuda()
    for alpha in (0.001, 1e-4):
        want = ref.linear_a8_w8_b8_o8(x, w, b, alpha, 0.01)
        assert_bit_exact(cuda_ops.linear_a8_w8_b8_o8(x, w, b, alpha, 0.01), want, f"b8_o8 alpha={alpha}")
        want = ref.linear_relu_a8_w8_b8_o8(x, w, b, alpha, 0.01)
        assert_bit_exact(cuda_ops.linear_relu_a8_w8_b8_o8(x, w, b, alpha, 0.01), want, f"relu alpha={alpha}")


@pytest.mark.parametrize("m,n,k", [(128, 1024, 512), (77, 272, 144), (300, 528, 400), (16, 7168, 7168), (2048, 5120, 5120)])
def test_all_linear_ops_vs_reference_kernels(cuda_ops, ref, m, n, k):
    C = cuda_ops
    x, w = rand_s8((m, k), m + n).cuda(), rand_s8((n, k), k).cuda()
    b8, b32, bf = rand_s8((n,), 1).cuda(), rand_s32((n,), 2).cuda(), randn((n,), 3).cuda()
    alpha, beta = 1.0 / (60.0 * k ** 0.5), 0.01
    assert_bit_exact(C.linear_a8_w8_b32_o32(x, w, b32), ref.linear_a8_w8_b32_o32(x, w, b32), "b32_o32")
    assert_bit_exact(C.linear_a8_w8_b8_o8(x, w, b8, alpha, beta), ref.linear_a8_w8_b8_o8(x, w, b8, alpha, beta), "b8_o8")
    assert_bit_exact(C.linear_relu_a8_w8_b8_o8(x, w, b8, alpha, beta),
                     ref.linear_relu_a8_w8_b8_o8(x, w, b8, alpha, beta), "relu_b8_o8")
    assert_fp32_close(C.linear_a8_w8_bfp32_ofp32(x, w, bf, alpha, 1.0), ref.linear_a8_w8_bfp32_ofp32(x, w, bf, alpha, 1.0),
                      1e-5, "bfp32_ofp32")
    assert_bit_exact(C.linear_a8_w8_b32_o32_with_scaling(x, w, b32, alpha, beta * 1e-7),
                     ref.linear_a8_w8_b32_o32_with_scaling(x, w, b32, alpha, beta * 1e-7), "b32_o32_with_scaling")


@pytest.mark.parametrize("batch,m,n,k", [(6, 48, 48, 128), (4, 512, 512, 128), (3, 200, 128, 208)])
def test_bmm_ops_vs_reference_kernels(cuda_ops, ref, batch, m, n, k):
    C = cuda_ops
    a, b = rand_s8((batch, m, k), 5).cuda(), rand_s8((batch, n, k), 6).cuda()
    assert_bit_exact(C.bmm_s8t_s8n_s32t(a, b), ref.bmm_s8t_s8n_s32t(a, b), "s32t")
    assert_fp32_close(C.bmm_s8t_s8n_f32t(a, b, 1.0 / 127 ** 2), ref.bmm_s8t_s8n_f32t(a, b, 1.0 / 127 ** 2), 1e-5, "f32t")
    assert_bit_exact(C.bmm_s8t_s8n_s8t(a, b, 2e-4), ref.bmm_s8t_s8n_s8t(a, b, 2e-4), "s8t")
