"""The oracle's dq_add_layernorm_q against the REFERENCE's own C++ implementation
(torch_int/kernels/fused.cu), compiled from the reference checkout by oracle/build_ref.py into
oracle/_ref/ref_fused.so and run on CPU tensors as the reference's tests/test_dq_add_ln_q.py does.
Skipped when the module has not been built (no reference checkout on this machine)."""
import pytest
import torch

from oracle import build_ref
from oracle import w8a8 as O


@pytest.fixture(scope="module")
def ref():
    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref/ref_fused.so is not built (python oracle/build_ref.py <reference checkout>)")
    return mod


@pytest.mark.parametrize("shape,scale,gs", [((2, 3, 4), 0.01, 1.0), ((3, 17, 256), 0.003, 12.0), ((2, 64, 5120), 1e-5, 30.0),
                                            ((1, 16, 12288), 2e-5, 25.0), ((5, 90), 0.02, 3.0)])
def test_oracle_equals_reference_cpp(ref, shape, scale, gs):
    g = torch.Generator().manual_seed(hash(shape) % 1000)
    h = shape[-1]
    x = torch.randint(-200000, 200000, shape, generator=g, dtype=torch.int32)
    res = torch.randn(shape, generator=g)
    gamma = (1.0 + 0.1 * torch.randn(h, generator=g)) * gs
    beta = 0.1 * torch.randn(h, generator=g) * gs
    keep_res = res.clone()
    r_ref, q_ref = ref.dq_add_layernorm_q(x, scale, res, gamma, beta, 1e-5)
    r, q = O.dq_add_layernorm_q(x, scale, res, gamma, beta, 1e-5)
    assert q_ref.dtype == torch.int8 and r_ref.dtype == res.dtype
    assert torch.equal(r, r_ref), "residual output"
    assert torch.equal(q, q_ref), "int8 LayerNorm output"
    assert torch.equal(res, keep_res), "the reference does not modify its residual input (fused.cu:17)"


def test_reference_cpp_saturates_and_rounds_half_to_even(ref):
    # gamma large enough that LayerNorm outputs leave the int8 range; beta chosen to create exact .5 ties
    x = torch.zeros((1, 4), dtype=torch.int32)
    res = torch.tensor([[-1.0, 1.0, -1.0, 1.0]])
    for gamma_v, beta_v, want in ((1000.0, 0.0, [-128, 127, -128, 127]), (1.0, 1.5, [0, 2, 0, 2]), (2.0, 0.5, [-2, 2, -2, 2])):
        gamma, beta = torch.full((4,), gamma_v), torch.full((4,), beta_v)
        _, q_ref = ref.dq_add_layernorm_q(x, 1.0, res, gamma, beta, 0.0)
        _, q = O.dq_add_layernorm_q(x, 1.0, res, gamma, beta, 0.0)
        assert torch.equal(q, q_ref)
        assert q_ref.view(-1).tolist() == want
