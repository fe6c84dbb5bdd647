"""Shared helpers of the test-suite: seeded inputs and comparison rules."""
import torch


def rand_s8(shape, seed, lo=-127, hi=127):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, shape, generator=g, dtype=torch.int8)


def rand_s32(shape, seed, lo=-2 ** 31, hi=2 ** 31 - 1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi, shape, generator=g, dtype=torch.int32)


def randn(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def assert_bit_exact(got, want, what=""):
    got, want = got.cpu(), want.cpu()
    assert got.dtype == want.dtype and got.shape == want.shape, (what, got.dtype, want.dtype, got.shape, want.shape)
    if not torch.equal(got, want):
        d = (got.to(torch.int64) - want.to(torch.int64)).abs()
        raise AssertionError(f"{what}: {int((d != 0).sum())} of {d.numel()} elements differ, max |d| = {int(d.max())}")


def assert_fp32_close(got, want, rel=1e-5, what=""):
    """fp32 outputs: within `rel` relative (the bar stated for this path)."""
    got, want = got.cpu().double(), want.cpu().double()
    err = (got - want).abs()
    tol = rel * want.abs().clamp_min(1e-30) + 1e-30
    bad = err > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} elements beyond {rel} relative, max rel err " \
                          f"{float((err / want.abs().clamp_min(1e-30)).max()):.3g}"


def assert_quant_close(got, want, min_exact=0.999, what=""):
    """int8 outputs of LayerNorm / softmax paths: the fp32 reduction order may
    differ from torch's, which can flip a value only at a rounding tie: at
    most 1 LSB anywhere and at least `min_exact` of all elements identical."""
    got, want = got.cpu().to(torch.int32), want.cpu().to(torch.int32)
    d = (got - want).abs()
    exact = float((d == 0).double().mean())
    assert int(d.max()) <= 1, f"{what}: max |d| = {int(d.max())}"
    assert exact >= min_exact, f"{what}: only {exact:.5f} of elements identical"


def set_residual_in_gemm(model, on):
    """Switches every decoder layer of `model` between adding the out_proj / fc2 outputs to the residual in
    the GEMM epilogue and in the fused residual/LayerNorm row kernel (bit-identical results)."""
    for m in model.modules():
        if hasattr(m, "residual_in_gemm"):
            m.residual_in_gemm = bool(on)
    return model


def set_fused_attention(model, on):
    """Switches every attention module of `model` between the one-kernel causal attention and the
    scores -> softmax_q -> context chain (the two agree except at rounding ties of a probability)."""
    for m in model.modules():
        if hasattr(m, "fused_attention"):
            m.fused_attention = bool(on)
    return model
