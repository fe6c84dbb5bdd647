"""TEST INFRASTRUCTURE: CPU oracle of the reference's W8A8 operator set.

One function per op the reference exports from ``torch_int._CUDA``
(torch_int/kernels/bindings.cpp:5-20), plus the torch-only pieces of the path
(``LayerNormQ.forward``, the softmax->int8 chain of ``Int8OPTAttention``).
Inputs and outputs are CPU torch tensors with the reference's shapes.

The integer contraction and the fp32 epilogues run in the C restatement
(``w8a8_oracle.c``: exact int32 accumulation, single-rounded ``fmaf``);
``*_numpy`` twins restate the same arithmetic in numpy (int64 matmul, FMA
emulated through float64) and are used to cross-check the C code.  The
LayerNorm / softmax pieces call the very torch functions the reference calls.

Pinned by tests/golden (fixtures generated from the reference's importable
Python code and from the formulas of its tests); the last-bit rounding order of
the GEMM epilogues is pinned only by CUTLASS's documented semantics ("parity
unpinned" there, see w8a8_oracle.c).

Never imported by the product.
"""
import ctypes
import os

import numpy as np
import torch

from . import build as _build

_lib = None


def lib():
    """Loads (building first if needed) the C oracle."""
    global _lib
    if _lib is None:
        path = _build.OUT
        if not os.path.exists(path):
            path = _build.build()
        L = ctypes.CDLL(path)
        p, i64, f32, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int
        L.ti_oracle_gemm_acc.argtypes = [p, p, p, i64, i64, i64, i64]
        L.ti_oracle_gemm_acc_naive.argtypes = [p, p, p, i64, i64, i64, i64]
        L.ti_oracle_epi_s8_bias_s8.argtypes = [p, p, p, i64, i64, f32, f32, i32]
        L.ti_oracle_epi_f32_bias_f32.argtypes = [p, p, p, i64, i64, f32, f32]
        L.ti_oracle_epi_s32_bias_s32_add.argtypes = [p, p, p, i64, i64]
        L.ti_oracle_epi_s32_bias_s32_scale.argtypes = [p, p, p, i64, i64, f32, f32]
        L.ti_oracle_epi_f32_alpha.argtypes = [p, p, i64, f32]
        L.ti_oracle_epi_s8_alpha.argtypes = [p, p, i64, f32]
        L.ti_oracle_num_threads.restype = ctypes.c_int
        for name in ("ti_oracle_gemm_acc", "ti_oracle_gemm_acc_naive", "ti_oracle_epi_s8_bias_s8",
                     "ti_oracle_epi_f32_bias_f32", "ti_oracle_epi_s32_bias_s32_add",
                     "ti_oracle_epi_s32_bias_s32_scale", "ti_oracle_epi_f32_alpha",
                     "ti_oracle_epi_s8_alpha"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def num_threads():
    """Host threads the C oracle's OpenMP loops use."""
    return lib().ti_oracle_num_threads()


def _c(t, dtype):
    assert t.device.type == "cpu", "the oracle works on CPU tensors"
    assert t.dtype == dtype, f"expected {dtype}, got {t.dtype}"
    return t.contiguous()


# ------------------------------------------------------------------ contraction
def gemm_acc(a, b, naive=False):
    """int32 acc[..., m, n] = sum_k a[..., m, k] * b[..., n, k]; a, b int8, 2-D or 3-D.
    The contraction of every linear/bmm op (linear.cu:30-32, bmm.cu:22-24)."""
    a, b = _c(a, torch.int8), _c(b, torch.int8)
    squeeze = a.dim() == 2
    if squeeze:
        a, b = a.unsqueeze(0), b.unsqueeze(0)
    batch, m, k = a.shape
    bb, n, kb = b.shape
    assert bb == batch and kb == k
    out = torch.empty((batch, m, n), dtype=torch.int32)
    fn = lib().ti_oracle_gemm_acc_naive if naive else lib().ti_oracle_gemm_acc
    fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, m, n, k)
    return out[0] if squeeze else out


def gemm_acc_numpy(a, b):
    """Same contraction with numpy int64 matmul (slow; small shapes only)."""
    an, bn = a.numpy().astype(np.int64), b.numpy().astype(np.int64)
    acc = an @ np.swapaxes(bn, -1, -2)
    return torch.from_numpy(acc.astype(np.int32))


def gemm_acc_fp64(a, b):
    """Same contraction through float64 BLAS: exact because K * 128^2 < 2^53."""
    acc = a.double() @ b.double().transpose(-1, -2)
    return acc.round().to(torch.int64).to(torch.int32)


# -------------------------------------------------------------------- epilogues
def _bias(bias, n, dtype):
    return _c(bias.reshape(-1), dtype) if bias.numel() == n else None


def linear_a8_w8_b8_o8(x, w, bias, alpha, beta, relu=False):
    """int8 y = sat_rne(fma(alpha, f32(acc), beta * f32(bias))) (linear.cu:369-473)."""
    acc = gemm_acc(x, w)
    m, n = acc.shape
    b = _bias(bias, n, torch.int8)
    out = torch.empty((m, n), dtype=torch.int8)
    lib().ti_oracle_epi_s8_bias_s8(acc.data_ptr(), b.data_ptr(), out.data_ptr(), m, n,
                                   float(alpha), float(beta), 1 if relu else 0)
    return out


def epilogue_s8_bias_s8(acc, bias, alpha, beta, relu=False):
    """The int8 epilogue of linear_a8_w8_b8_o8 / linear_relu_a8_w8_b8_o8 applied to given int32
    accumulators [M, N] (the C restatement; for callers that already hold the contraction)."""
    acc = _c(acc, torch.int32)
    m, n = acc.shape
    b = _bias(bias, n, torch.int8)
    out = torch.empty((m, n), dtype=torch.int8)
    lib().ti_oracle_epi_s8_bias_s8(acc.data_ptr(), b.data_ptr(), out.data_ptr(), m, n,
                                   float(alpha), float(beta), 1 if relu else 0)
    return out


def linear_relu_a8_w8_b8_o8(x, w, bias, alpha, beta):
    """linear_a8_w8_b8_o8 with max(y, 0) before rounding (linear.cu:476-625)."""
    return linear_a8_w8_b8_o8(x, w, bias, alpha, beta, relu=True)


def linear_a8_w8_bfp32_ofp32(x, w, bias, alpha, beta):
    """fp32 y = fma(alpha, f32(acc), beta * bias) (linear.cu:246-365)."""
    acc = gemm_acc(x, w)
    m, n = acc.shape
    b = _bias(bias, n, torch.float32)
    out = torch.empty((m, n), dtype=torch.float32)
    lib().ti_oracle_epi_f32_bias_f32(acc.data_ptr(), b.data_ptr(), out.data_ptr(), m, n,
                                     float(alpha), float(beta))
    return out


def linear_a8_w8_b32_o32(x, w, bias):
    """int32 y = acc + bias with two's-complement wrap (linear.cu:13-136)."""
    acc = gemm_acc(x, w)
    m, n = acc.shape
    b = _bias(bias, n, torch.int32)
    out = torch.empty((m, n), dtype=torch.int32)
    lib().ti_oracle_epi_s32_bias_s32_add(acc.data_ptr(), b.data_ptr(), out.data_ptr(), m, n)
    return out


def linear_a8_w8_b32_o32_with_scaling(x, w, bias, alpha, beta):
    """int32 y = sat_rne(fma(alpha, f32(acc), beta * f32(bias))) (linear.cu:139-243)."""
    acc = gemm_acc(x, w)
    m, n = acc.shape
    b = _bias(bias, n, torch.int32)
    out = torch.empty((m, n), dtype=torch.int32)
    lib().ti_oracle_epi_s32_bias_s32_scale(acc.data_ptr(), b.data_ptr(), out.data_ptr(), m, n,
                                           float(alpha), float(beta))
    return out


def bmm_s8t_s8n_f32t(a, b, alpha):
    """fp32 C[b] = alpha * f32(acc) (bmm.cu:10-108)."""
    acc = gemm_acc(a, b)
    out = torch.empty(acc.shape, dtype=torch.float32)
    lib().ti_oracle_epi_f32_alpha(acc.data_ptr(), out.data_ptr(), acc.numel(), float(alpha))
    return out


def bmm_s8t_s8n_s8t(a, b, alpha):
    """int8 C[b] = sat_rne(alpha * f32(acc)) (bmm.cu:110-208)."""
    acc = gemm_acc(a, b)
    out = torch.empty(acc.shape, dtype=torch.int8)
    lib().ti_oracle_epi_s8_alpha(acc.data_ptr(), out.data_ptr(), acc.numel(), float(alpha))
    return out


def bmm_s8t_s8n_s32t(a, b):
    """int32 C[b] = acc (bmm.cu:210-295)."""
    return gemm_acc(a, b)


# ------------------------------------------------- numpy twins of the epilogues
def _f32(v):
    return np.float32(v)


def _fma32(alpha, a, t):
    """fp32 fma(alpha, a, t) emulated through float64: the product of two
    float32 values is exact in float64; one rounding of the sum to float64 and
    one to float32 (differs from a true FMA only in rare double-rounding cases)."""
    return (np.float64(alpha) * a.astype(np.float64) + t.astype(np.float64)).astype(np.float32)


def _rne_sat(y, lo, hi, dtype):
    r = np.rint(y.astype(np.float64))  # rint = round half to even; float32 -> float64 is exact
    return np.clip(r, lo, hi).astype(dtype)


def epilogue_numpy(acc, bias, alpha, beta, kind):
    """numpy restatement of every epilogue; `kind` is the op name suffix."""
    a = acc.numpy().astype(np.float32)  # int32 -> float32, round to nearest
    alpha, beta = _f32(alpha), _f32(beta)
    if kind in ("b8_o8", "relu_b8_o8", "b32_o32_with_scaling", "bfp32_ofp32"):
        t = (beta * bias.reshape(-1).numpy().astype(np.float32)).astype(np.float32)
        y = _fma32(alpha, a, np.broadcast_to(t, a.shape))
        if kind == "relu_b8_o8":
            y = np.maximum(y, np.float32(0))
        if kind == "bfp32_ofp32":
            return torch.from_numpy(y)
        if kind == "b32_o32_with_scaling":
            return torch.from_numpy(_rne_sat(y, -2 ** 31, 2 ** 31 - 1, np.int32))
        return torch.from_numpy(_rne_sat(y, -128, 127, np.int8))
    if kind == "b32_o32":
        s = acc.numpy().astype(np.int64) + bias.reshape(-1).numpy().astype(np.int64)
        return torch.from_numpy(((s + 2 ** 31) % 2 ** 32 - 2 ** 31).astype(np.int32))
    if kind == "f32t":
        return torch.from_numpy((alpha * a).astype(np.float32))
    if kind == "s8t":
        return torch.from_numpy(_rne_sat((alpha * a).astype(np.float32), -128, 127, np.int8))
    if kind == "s32t":
        return acc.clone()
    raise ValueError(kind)


# ------------------------------------------------------- LayerNorm-quantise ops
def layernorm_q(x, gamma, beta, eps):
    """LayerNormQ.forward (torch_int/nn/fused.py:13-18): cast to the parameters'
    dtype, layer_norm, round, clamp, int8 - with the same torch calls."""
    x = x.to(gamma.dtype)
    ln = torch.nn.functional.layer_norm(x, x.shape[-1:], gamma, beta, eps)
    return ln.round().clamp(-128, 127).to(torch.int8)


def dq_add_layernorm_q(input_int32, input_scale, residual, gamma, beta, eps):
    """dq_add_layernorm_q (torch_int/kernels/fused.cu:17-23, same as
    functional/fused.py:5-12): torch.add with alpha, layer_norm, clamp, round, int8."""
    r = torch.add(residual, input_int32, alpha=input_scale)
    ln = torch.nn.functional.layer_norm(r, r.shape[-1:], gamma, beta, eps)
    return r, ln.clamp(-128, 127).round().to(torch.int8)


def dq_add_layernorm_q_bias(input_int32, input_scale, input_bias, residual, gamma, beta, eps):
    """Extension used after an int32 all-reduce: d = fma(scale, f32(in), bias) as
    the fp32-output linear computes it (linear.cu:246-365), then residual + d,
    then LayerNormQ."""
    a = input_int32.numpy().astype(np.float32)
    d = _fma32(_f32(input_scale), a, np.broadcast_to(input_bias.numpy().astype(np.float32), a.shape))
    # residual.add_(d.to(residual.dtype)) of the decoder layer (models/opt.py:281,289), then LayerNormQ,
    # which casts to its parameters' dtype first (nn/fused.py:14)
    r = residual + torch.from_numpy(d).to(residual.dtype)
    ln = torch.nn.functional.layer_norm(r.to(gamma.dtype), r.shape[-1:], gamma, beta, eps)
    return r, ln.clamp(-128, 127).round().to(torch.int8)


def softmax_q(scores, mask=None):
    """The probability path of Int8OPTAttention.forward (torch_int/models/opt.py:
    139-178): scores [B*H,T,S] fp32 (+ mask [B,1,T,S] viewed per head), floor at
    finfo.min, softmax, * 127, round, int8."""
    s = scores
    if mask is not None:
        bh, t, src = scores.shape
        bsz = mask.shape[0]
        s = s.view(bsz, bh // bsz, t, src) + mask.view(bsz, 1, t, src)
        s = torch.max(s, torch.tensor(torch.finfo(s.dtype).min))
        s = s.view(bh, t, src)
    p = torch.nn.functional.softmax(s, dim=-1)
    p = p.mul(127).round()
    return p.to(torch.int8)


def causal_mask(bsz, tgt, src, dtype=torch.float32):
    """Additive causal mask [bsz,1,tgt,src] with finfo.min above the diagonal
    (what transformers' OPT decoder builds for the reference; the last `tgt`
    source positions are the current tokens)."""
    m = torch.full((tgt, src), torch.finfo(dtype).min, dtype=dtype)
    past = src - tgt
    m = torch.triu(m, diagonal=past + 1)
    return m.view(1, 1, tgt, src).expand(bsz, 1, tgt, src).contiguous()
