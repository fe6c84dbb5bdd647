"""Drop-in for the reference's native extension module ``torch_int._CUDA``.

Exports the nine callables of the reference's pybind11 module with the same
names, positional arguments and return values
(torch_int/kernels/bindings.cpp:5-20), implemented by the sm_100a kernels of
``libtorch_int_b200.so`` through its C ABI (include/torch_int_b200.h).  This
shim only validates tensors, allocates the output, looks up the device and the
current stream and forwards raw pointers; it never computes anything itself
and there is no CPU or PyTorch fallback: importing it without the built
library, or calling an op with a CPU tensor, raises.

Differences from the reference wrappers, all deliberate:
  * inputs are validated (dtype, device, contiguity, shape agreement) and a
    ``RuntimeError`` is raised where the reference would silently compute on
    assumed-packed strides (torch_int/kernels/linear.cu:429-434);
  * kernels run on the current stream of the input's device instead of the
    legacy default stream of the current device;
  * the bias is read as a vector, no M x N matrix is materialised
    (torch_int/kernels/linear.cu:83,420).
Extra callables (not in the reference) are listed at the end of ``__all__``.
"""
import ctypes
import os

import torch

__all__ = [
    "linear_a8_w8_b8_o8", "linear_relu_a8_w8_b8_o8", "linear_a8_w8_bfp32_ofp32",
    "linear_a8_w8_b32_o32", "linear_a8_w8_b32_o32_with_scaling",
    "bmm_s8t_s8n_s8t", "bmm_s8t_s8n_f32t", "bmm_s8t_s8n_s32t", "dq_add_layernorm_q",
    # extras
    "layernorm_q", "softmax_q", "dq_add_layernorm_q_bias", "gemm_i8_ex", "transpose_values", "device_status",
    "library_path",
]

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libtorch_int_b200.so")


def library_path():
    """Path of the shared library this module forwards to."""
    return _LIB_PATH


if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"torch_int._CUDA: {_LIB_PATH} is missing; build it with "
        "`python torch-int_b200/csrc/build.py` (needs nvcc with sm_100a support). "
        "There is no fallback implementation.")

_lib = ctypes.CDLL(_LIB_PATH)

_i64, _f32, _i32, _ptr = ctypes.c_int64, ctypes.c_float, ctypes.c_int, ctypes.c_void_p


class _GemmDesc(ctypes.Structure):
    # struct ti_gemm_desc (include/torch_int_b200.h)
    _fields_ = [
        ("A", _ptr), ("B", _ptr), ("C", _ptr), ("bias", _ptr),
        ("M", _i64), ("N", _i64), ("K", _i64),
        ("batch", _i64), ("batch2", _i64),
        ("lda", _i64), ("ldb", _i64), ("ldc", _i64),
        ("strideA", _i64), ("strideB", _i64), ("strideC", _i64),
        ("stride2A", _i64), ("stride2B", _i64), ("stride2C", _i64),
        ("alpha", _f32), ("beta", _f32),
        ("epilogue", ctypes.c_int32), ("tile_n", ctypes.c_int32), ("cta_pair", ctypes.c_int32),
        ("scatter_rows", _i64), ("scatter_ptrs", _ptr * 8),
        ("alpha_vec", _ptr), ("beta_vec", _ptr),
        ("workspace", _ptr), ("workspace_bytes", _i64), ("splits", ctypes.c_int32),
    ]


def _sig(name, argtypes, restype=ctypes.c_int):
    fn = getattr(_lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


_linear_sig = [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _f32, _f32, _ptr]
_c_linear_b8_o8 = _sig("ti_linear_a8_w8_b8_o8", _linear_sig)
_c_linear_relu_b8_o8 = _sig("ti_linear_relu_a8_w8_b8_o8", _linear_sig)
_c_linear_bfp32_ofp32 = _sig("ti_linear_a8_w8_bfp32_ofp32", _linear_sig)
_c_linear_b32_o32 = _sig("ti_linear_a8_w8_b32_o32", [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _ptr])
_c_linear_b32_o32_scaling = _sig("ti_linear_a8_w8_b32_o32_with_scaling", _linear_sig)
_bmm_sig = [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _f32, _ptr]
_c_bmm_f32 = _sig("ti_bmm_s8t_s8n_f32t", _bmm_sig)
_c_bmm_s8 = _sig("ti_bmm_s8t_s8n_s8t", _bmm_sig)
_c_bmm_s32 = _sig("ti_bmm_s8t_s8n_s32t", [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr])
_c_gemm_ex = _sig("ti_gemm_i8_ex", [ctypes.POINTER(_GemmDesc), _ptr])
_c_dq_add_ln_q = _sig("ti_dq_add_layernorm_q",
                      [_ptr, _f32, _ptr, _i32, _ptr, _ptr, _f32, _ptr, _ptr, _i64, _i64, _ptr])
_c_dq_add_ln_q_bias = _sig("ti_dq_add_layernorm_q_bias",
                           [_ptr, _f32, _ptr, _ptr, _i32, _ptr, _ptr, _f32, _ptr, _ptr, _i64, _i64, _ptr])
_c_ln_q = _sig("ti_layernorm_q", [_ptr, _i32, _ptr, _ptr, _f32, _ptr, _i64, _i64, _ptr])
_c_softmax_q = _sig("ti_softmax_q", [_ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _ptr])
_c_tp_reduce_ln_q = _sig("ti_tp_reduce_layernorm_q",
                          [_ptr, _i32, _i64, _f32, _ptr, _ptr, _ptr, _ptr, _f32, _ptr, ctypes.POINTER(_ptr), _i32,
                           _i64, _i64, _i64, _ptr])
_c_tp_barrier = _sig("ti_tp_barrier_limit", [ctypes.POINTER(_ptr), _i32, _i32, ctypes.c_uint32, _i64, _ptr])
_c_tp_exchange_reduce_ln_q = _sig("ti_tp_exchange_reduce_layernorm_q",
                                  [_ptr, _i32, _i64, _f32, _ptr, _ptr, _ptr, _ptr, _f32, _ptr, ctypes.POINTER(_ptr),
                                   _i32, _i64, _i64, _i64, ctypes.POINTER(_ptr), _i32, _i32, ctypes.c_uint32, _ptr,
                                   _i64, _ptr])
_c_decode_attention = _sig("ti_decode_attention_s8",
                           [_ptr, _i64, _ptr, _ptr, _i64, _i64, _i64, _i64, _ptr, _f32, _f32, _ptr, _i64, _ptr])
_c_advance_position = _sig("ti_advance_position", [_ptr, _i32, _ptr])
_c_attention_prefill = _sig("ti_attention_prefill_s8",
                            [_ptr, _i64, _i64, _ptr, _i64, _i64, _ptr, _i64, _ptr, _i64, _i64,
                             _i64, _i64, _i64, _i64, _i64, _f32, _f32, _ptr])
_c_transpose_values = _sig("ti_transpose_values", [_ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _ptr])
_c_last_error = _sig("ti_last_error", [], ctypes.c_char_p)
_c_device_status = _sig("ti_device_status", [ctypes.POINTER(ctypes.c_int), _i32])
_c_abi_version = _sig("ti_abi_version", [])
_c_set_sm_limit = _sig("ti_set_sm_limit", [_i32])
_c_set_group_m = _sig("ti_set_group_m", [_i32])
_c_set_dependent_launch = _sig("ti_set_dependent_launch", [_i32])
_c_set_narrow_a = _sig("ti_set_narrow_a", [_i32])

if _c_abi_version() != 1:
    raise ImportError("torch_int._CUDA: libtorch_int_b200.so has an unexpected ABI version")

EPI_S8_BIAS_S8, EPI_S8_BIAS_S8_RELU, EPI_F32_BIAS_F32, EPI_S32_BIAS_S32_ADD, \
    EPI_S32_BIAS_S32_SCALE, EPI_F32_ALPHA, EPI_S8_ALPHA, EPI_S32_RAW, EPI_S8_BIAS_S8_VEC, \
    EPI_F32_BIAS_F32_ACC = range(10)
_EPI_OUT_DTYPE = {
    EPI_S8_BIAS_S8: torch.int8, EPI_S8_BIAS_S8_RELU: torch.int8, EPI_F32_BIAS_F32: torch.float32,
    EPI_S32_BIAS_S32_ADD: torch.int32, EPI_S32_BIAS_S32_SCALE: torch.int32,
    EPI_F32_ALPHA: torch.float32, EPI_S8_ALPHA: torch.int8, EPI_S32_RAW: torch.int32,
    EPI_S8_BIAS_S8_VEC: torch.int8, EPI_F32_BIAS_F32_ACC: torch.float32,
}
_EPI_BIAS_DTYPE = {
    EPI_S8_BIAS_S8: torch.int8, EPI_S8_BIAS_S8_RELU: torch.int8, EPI_F32_BIAS_F32: torch.float32,
    EPI_S32_BIAS_S32_ADD: torch.int32, EPI_S32_BIAS_S32_SCALE: torch.int32, EPI_S8_BIAS_S8_VEC: torch.int8,
    EPI_F32_BIAS_F32_ACC: torch.float32,
}


_SPLIT_K_MAX_ROWS = 128            # split-K applies to problems with at most one M tile
_SPLIT_K_WORKSPACE_BYTES = 32 << 20  # per-device scratch of the split-K path (covers M x N <= 8M)
_workspaces = {}


def _split_k_workspace(device):
    """Zero-initialised scratch the split-K GEMM path accumulates into (one per device; every
    launch leaves it zeroed).  Launches that use it must not overlap on the GPU: all of this
    module's GEMMs of one device are expected on one stream at a time."""
    ws = _workspaces.get(device.index)
    if ws is None:
        ws = torch.zeros(_SPLIT_K_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _workspaces[device.index] = ws
    return ws


split_k = True  # module switch: False disables the split-K path (every GEMM then needs no scratch)

launch_count = 0  # kernels of this library enqueued through this module since import


def _check(rc):
    global launch_count
    if rc != 0:
        raise RuntimeError("torch_int._CUDA: " + _c_last_error().decode("utf-8", "replace"))
    launch_count += 1


def _stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


class _on_device:
    """Makes `device` current for the duration of a call (cheap when it already is)."""

    __slots__ = ("idx", "prev")

    def __init__(self, device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def _require(t, name, dtype, ndim=None):
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this build has no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise RuntimeError(f"{name} must be {ndim}-dimensional, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous, got strides {t.stride()} for shape {tuple(t.shape)}")


def _bias_vector(bias, n, dtype, device):
    # The reference accepts any bias shape with N elements, on any device
    # (bias.to(device).view({1,-1}), torch_int/kernels/linear.cu:420).
    if not isinstance(bias, torch.Tensor):
        raise RuntimeError("bias must be a torch.Tensor")
    if bias.dtype != dtype:
        raise RuntimeError(f"bias must have dtype {dtype}, got {bias.dtype}")
    if bias.numel() != n:
        raise RuntimeError(f"bias must have {n} elements, got shape {tuple(bias.shape)}")
    if bias.device != device:
        bias = bias.to(device)
    return bias.reshape(-1).contiguous()


def _linear(cfn, epi, x, w, bias, bias_dtype, out_dtype, alpha=None, beta=None):
    _require(x, "input", torch.int8, 2)
    _require(w, "weight", torch.int8, 2)
    if w.device != x.device:
        raise RuntimeError("input and weight must be on the same device")
    m, k = x.shape
    n, kw = w.shape
    if k != kw:
        raise RuntimeError(f"input [{m},{k}] and weight [{n},{kw}] disagree on K")
    b = _bias_vector(bias, n, bias_dtype, x.device)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    if split_k and 0 < m <= _SPLIT_K_MAX_ROWS and k >= 2048:
        # few rows, long K (decode steps): the strided entry point can split K over the SMs
        return gemm_i8_ex(x, w, out, b, epilogue=epi, m=m, n=n, k=k, lda=k, ldb=k, ldc=n,
                          alpha=1.0 if alpha is None else alpha, beta=1.0 if beta is None else beta)
    with _on_device(x.device):
        s = _stream_ptr(x.device)
        if alpha is None:
            rc = cfn(x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, s)
        else:
            rc = cfn(x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k,
                     float(alpha), float(beta), s)
    _check(rc)
    return out


def linear_a8_w8_b8_o8(input, weight, bias, alpha, beta):
    """int8 [M,N] = sat_rne(alpha * (input . weight^T) + beta * bias); bias int8.
    Reference: torch_int/kernels/linear.cu:369-473."""
    return _linear(_c_linear_b8_o8, EPI_S8_BIAS_S8, input, weight, bias, torch.int8, torch.int8, alpha, beta)


def linear_relu_a8_w8_b8_o8(input, weight, bias, alpha, beta):
    """As linear_a8_w8_b8_o8 with ReLU before rounding.
    Reference: torch_int/kernels/linear.cu:476-625."""
    return _linear(_c_linear_relu_b8_o8, EPI_S8_BIAS_S8_RELU, input, weight, bias, torch.int8, torch.int8, alpha, beta)


def linear_a8_w8_bfp32_ofp32(input, weight, bias, alpha, beta):
    """fp32 [M,N] = alpha * (input . weight^T) + beta * bias; bias fp32.
    Reference: torch_int/kernels/linear.cu:246-365."""
    return _linear(_c_linear_bfp32_ofp32, EPI_F32_BIAS_F32, input, weight, bias, torch.float32, torch.float32, alpha, beta)


def linear_a8_w8_b32_o32(input, weight, bias):
    """int32 [M,N] = input . weight^T + bias; bias int32.
    Reference: torch_int/kernels/linear.cu:13-136."""
    return _linear(_c_linear_b32_o32, EPI_S32_BIAS_S32_ADD, input, weight, bias, torch.int32, torch.int32)


def linear_a8_w8_b32_o32_with_scaling(input, weight, bias, alpha, beta):
    """int32 [M,N] = sat_rne(alpha * (input . weight^T) + beta * bias); bias int32.
    Reference: torch_int/kernels/linear.cu:139-243."""
    return _linear(_c_linear_b32_o32_scaling, EPI_S32_BIAS_S32_SCALE, input, weight, bias, torch.int32, torch.int32, alpha, beta)


def _bmm(cfn, a, b, out_dtype, alpha=None):
    _require(a, "A", torch.int8, 3)
    _require(b, "B", torch.int8, 3)
    if a.device != b.device:
        raise RuntimeError("A and B must be on the same device")
    batch, m, k = a.shape
    bb, n, kb = b.shape
    if bb != batch or kb != k:
        raise RuntimeError(f"A {tuple(a.shape)} and B {tuple(b.shape)} must be [B,M,K] and [B,N,K]")
    out = torch.empty((batch, m, n), dtype=out_dtype, device=a.device)
    with _on_device(a.device):
        s = _stream_ptr(a.device)
        if alpha is None:
            rc = cfn(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, m, n, k, s)
        else:
            rc = cfn(a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, m, n, k, float(alpha), s)
    _check(rc)
    return out


def bmm_s8t_s8n_s8t(A, B, alpha):
    """int8 [B,M,N] = sat_rne(alpha * A[b] . B[b]^T).  Reference: torch_int/kernels/bmm.cu:110-208."""
    return _bmm(_c_bmm_s8, A, B, torch.int8, alpha)


def bmm_s8t_s8n_f32t(A, B, alpha):
    """fp32 [B,M,N] = alpha * A[b] . B[b]^T.  Reference: torch_int/kernels/bmm.cu:10-108."""
    return _bmm(_c_bmm_f32, A, B, torch.float32, alpha)


def bmm_s8t_s8n_s32t(A, B):
    """int32 [B,M,N] = A[b] . B[b]^T.  Reference: torch_int/kernels/bmm.cu:210-295."""
    return _bmm(_c_bmm_s32, A, B, torch.int32)


def _float_kind(t, name):
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.float16:
        return 1
    raise RuntimeError(f"{name} must be float32 or float16, got {t.dtype}")


def _affine(gamma, beta, h, device):
    # gamma/beta are fp32 buffers in the reference modules (torch_int/nn/fused.py:10-11).
    out = []
    for t, name in ((gamma, "gamma"), (beta, "beta")):
        if not isinstance(t, torch.Tensor) or t.numel() != h:
            raise RuntimeError(f"{name} must be a tensor with {h} elements")
        t = t.detach()
        if t.device != device or t.dtype != torch.float32 or not t.is_contiguous():
            t = t.to(device=device, dtype=torch.float32).contiguous()
        out.append(t.reshape(-1))
    return out


def dq_add_layernorm_q(input, input_scale, residual_input, gamma, beta, epsilon):
    """(residual_out, ln_out int8) = dequant-add-LayerNorm-quant in one kernel.
    Reference: torch_int/kernels/fused.cu:7-25."""
    return dq_add_layernorm_q_bias(input, input_scale, None, residual_input, gamma, beta, epsilon)


def dq_add_layernorm_q_bias(input, input_scale, input_bias, residual_input, gamma, beta, epsilon):
    """dq_add_layernorm_q with an optional fp32 bias [H] added to the dequantised
    input before the residual add (no reference counterpart; used after an
    int32 all-reduce of row-parallel partial sums)."""
    _require(input, "input", torch.int32)
    _require(residual_input, "residual_input", None)
    kind = _float_kind(residual_input, "residual_input")
    if residual_input.shape != input.shape or input.device != residual_input.device:
        raise RuntimeError("input and residual_input must have the same shape and device")
    if input.dim() < 1:
        raise RuntimeError("input must have at least one dimension")
    h = input.shape[-1]
    rows = input.numel() // h if h else 0
    g, b = _affine(gamma, beta, h, input.device)
    res_out = torch.empty_like(residual_input)
    q = torch.empty(input.shape, dtype=torch.int8, device=input.device)
    with _on_device(input.device):
        s = _stream_ptr(input.device)
        if input_bias is None:
            rc = _c_dq_add_ln_q(input.data_ptr(), float(input_scale), residual_input.data_ptr(), kind,
                                g.data_ptr(), b.data_ptr(), float(epsilon), res_out.data_ptr(),
                                q.data_ptr(), rows, h, s)
        else:
            ib = _bias_vector(input_bias, h, torch.float32, input.device)
            rc = _c_dq_add_ln_q_bias(input.data_ptr(), float(input_scale), ib.data_ptr(),
                                     residual_input.data_ptr(), kind, g.data_ptr(), b.data_ptr(),
                                     float(epsilon), res_out.data_ptr(), q.data_ptr(), rows, h, s)
    _check(rc)
    return res_out, q


def layernorm_q(x, gamma, beta, epsilon, fp32_norm=True):
    """int8 = clamp(rne(LayerNorm(x) * gamma + beta)) in one kernel.
    Reference: LayerNormQ.forward, torch_int/nn/fused.py:13-18.  For fp16 x, fp32_norm=True normalises in
    fp32 (the reference with fp32 parameters: it casts x to their dtype first); False rounds the LayerNorm
    output to fp16 before quantising (the reference with parameters cast to fp16)."""
    _require(x, "x", None)
    kind = _float_kind(x, "x")
    if kind == 1 and fp32_norm:
        kind = 2
    h = x.shape[-1]
    rows = x.numel() // h if h else 0
    g, b = _affine(gamma, beta, h, x.device)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    with _on_device(x.device):
        rc = _c_ln_q(x.data_ptr(), kind, g.data_ptr(), b.data_ptr(), float(epsilon), q.data_ptr(),
                     rows, h, _stream_ptr(x.device))
    _check(rc)
    return q


def softmax_q(scores, mask=None, num_heads=1, causal=-1):
    """int8 probs = rne(127 * softmax(max(scores + mask, finfo.min))) over the last dim.
    scores fp32 [B*H, T, S]; mask: additive fp32 [B, 1, T, S] / [B, T, S] or None;
    causal >= 0 generates "column j visible iff j <= t + causal" instead.
    Reference: torch_int/models/opt.py:139-178."""
    _require(scores, "scores", torch.float32, 3)
    bh, t, s = scores.shape
    mptr = None
    if mask is not None:
        _require(mask, "mask", torch.float32)
        if mask.numel() != (bh // num_heads) * t * s or bh % num_heads != 0:
            raise RuntimeError(f"mask shape {tuple(mask.shape)} does not match scores {tuple(scores.shape)} "
                               f"with {num_heads} heads")
        mptr = mask.data_ptr()
    out = torch.empty((bh, t, s), dtype=torch.int8, device=scores.device)
    with _on_device(scores.device):
        rc = _c_softmax_q(scores.data_ptr(), mptr, out.data_ptr(), bh, num_heads, t, s, s, s,
                          int(causal), _stream_ptr(scores.device))
    _check(rc)
    return out


def gemm_i8_ex(a, b, out, bias=None, *, epilogue, m, n, k, batch=1, batch2=1, lda, ldb, ldc,
               stride_a=0, stride_b=0, stride_c=0, stride2_a=0, stride2_b=0, stride2_c=0,
               alpha=1.0, beta=0.0, tile_n=0, cta_pair=0, scatter_ptrs=None, scatter_rows=0,
               alpha_vec=None, beta_vec=None, splits=0):
    """Strided form (ti_gemm_i8_ex): operands are addressed through explicit
    element strides starting at each tensor's data pointer, so views can be
    multiplied without contiguous copies.  Writes into `out` and returns it.
    With scatter_ptrs (device addresses, possibly of peer GPUs) and scatter_rows, row
    block i of the output goes to scatter_ptrs[i] instead and `out` may be None."""
    for t, name in ((a, "a"), (b, "b")):
        if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.int8):
            raise RuntimeError(f"{name} must be a CUDA int8 tensor")
    if scatter_rows:
        return _gemm_scatter(a, b, bias, epilogue, m, n, k, lda, ldb, ldc, alpha, beta, tile_n, cta_pair,
                             scatter_ptrs, scatter_rows)
    if not (isinstance(out, torch.Tensor) and out.is_cuda and out.dtype == _EPI_OUT_DTYPE[epilogue]):
        raise RuntimeError(f"out must be a CUDA tensor of dtype {_EPI_OUT_DTYPE[epilogue]}")
    if a.device != b.device or a.device != out.device:
        raise RuntimeError("a, b and out must be on the same device")

    def _span(mm, kk, ld, nb, st, nb2, st2):
        return (mm - 1) * ld + kk + (nb - 1) * st + (nb2 - 1) * st2 if min(mm, kk, nb, nb2) > 0 else 0

    if _span(m, k, lda, batch, stride_a, batch2, stride2_a) > a.untyped_storage().nbytes() - a.storage_offset():
        raise RuntimeError("a: strides address memory beyond the tensor's storage")
    if _span(n, k, ldb, batch, stride_b, batch2, stride2_b) > b.untyped_storage().nbytes() - b.storage_offset():
        raise RuntimeError("b: strides address memory beyond the tensor's storage")
    if _span(m, n, ldc, batch, stride_c, batch2, stride2_c) > \
            out.untyped_storage().nbytes() // out.element_size() - out.storage_offset():
        raise RuntimeError("out: strides address memory beyond the tensor's storage")
    d = _GemmDesc()
    d.A, d.B, d.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    if epilogue in _EPI_BIAS_DTYPE:
        bv = _bias_vector(bias, n, _EPI_BIAS_DTYPE[epilogue], a.device)
        d.bias = bv.data_ptr()
    else:
        d.bias = None
    d.M, d.N, d.K, d.batch, d.batch2 = m, n, k, batch, batch2
    d.lda, d.ldb, d.ldc = lda, ldb, ldc
    d.strideA, d.strideB, d.strideC = stride_a, stride_b, stride_c
    d.stride2A, d.stride2B, d.stride2C = stride2_a, stride2_b, stride2_c
    d.alpha, d.beta, d.epilogue, d.tile_n, d.cta_pair = float(alpha), float(beta), epilogue, tile_n, cta_pair
    if epilogue == EPI_S8_BIAS_S8_VEC:
        for t, name in ((alpha_vec, "alpha_vec"), (beta_vec, "beta_vec")):
            if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.float32 and t.numel() == n
                    and t.is_contiguous()):
                raise RuntimeError(f"{name} must be a contiguous CUDA float32 tensor with {n} elements")
        d.alpha_vec, d.beta_vec = alpha_vec.data_ptr(), beta_vec.data_ptr()
    if split_k and m <= _SPLIT_K_MAX_ROWS and batch == 1 and batch2 == 1 and k >= 2048 \
            and 256 + m * n * 4 + n // 8 <= _SPLIT_K_WORKSPACE_BYTES:
        ws = _split_k_workspace(a.device)
        d.workspace, d.workspace_bytes, d.splits = ws.data_ptr(), ws.numel(), splits
    else:
        d.workspace, d.workspace_bytes, d.splits = None, 0, 1
    with _on_device(a.device):
        rc = _c_gemm_ex(ctypes.byref(d), _stream_ptr(a.device))
    _check(rc)
    return out


def _gemm_scatter(a, b, bias, epilogue, m, n, k, lda, ldb, ldc, alpha, beta, tile_n, cta_pair, ptrs, rows):
    if len(ptrs) * rows < m or len(ptrs) > 8:
        raise RuntimeError("scatter_ptrs must cover all rows with at most 8 blocks")
    d = _GemmDesc()
    d.A, d.B, d.C = a.data_ptr(), b.data_ptr(), None
    d.bias = _bias_vector(bias, n, _EPI_BIAS_DTYPE[epilogue], a.device).data_ptr() if epilogue in _EPI_BIAS_DTYPE else None
    d.M, d.N, d.K, d.batch, d.batch2 = m, n, k, 1, 1
    d.lda, d.ldb, d.ldc = lda, ldb, ldc
    d.alpha, d.beta, d.epilogue, d.tile_n, d.cta_pair = float(alpha), float(beta), epilogue, tile_n, cta_pair
    d.scatter_rows = rows
    for i, ptr in enumerate(ptrs):
        d.scatter_ptrs[i] = ptr
    with _on_device(a.device):
        rc = _c_gemm_ex(ctypes.byref(d), _stream_ptr(a.device))
    _check(rc)
    return None


def tp_reduce_layernorm_q(stage, n_partials, partial_stride, scale, bias, residual, gamma, beta, epsilon,
                          q_dst_ptrs, q_row_offset):
    """Tensor-parallel exchange, second half (ti_tp_reduce_layernorm_q): stage int32
    [n_partials, rows, H] (this rank's rows), residual fp32 [rows, H]; returns the new
    residual; the int8 LayerNorm output is written to the buffers at q_dst_ptrs."""
    _require(stage, "stage", torch.int32)
    _require(residual, "residual", torch.float32, 2)
    rows, h = residual.shape
    g, b = _affine(gamma, beta, h, residual.device)
    ib = _bias_vector(bias, h, torch.float32, residual.device)
    out = torch.empty_like(residual)
    arr = (_ptr * len(q_dst_ptrs))(*q_dst_ptrs)
    with _on_device(residual.device):
        rc = _c_tp_reduce_ln_q(stage.data_ptr(), n_partials, partial_stride, float(scale), ib.data_ptr(),
                               residual.data_ptr(), g.data_ptr(), b.data_ptr(), float(epsilon), out.data_ptr(),
                               arr, len(q_dst_ptrs), q_row_offset, rows, h, _stream_ptr(residual.device))
    _check(rc)
    return out


def tp_exchange_reduce_layernorm_q(stage, n_partials, partial_stride, scale, bias, residual, gamma, beta, epsilon,
                                   q_dst_ptrs, q_row_offset, pad_ptrs, rank, epoch, counter, limit_ms=2000):
    """tp_reduce_layernorm_q with the exchange's synchronisation inside the kernel
    (ti_tp_exchange_reduce_layernorm_q): announces this rank's partial sums, waits for all ranks', reduces,
    and returns (in stream order) only when every rank's reduction is complete.  `counter`: an int32 CUDA
    tensor with one zero element, reserved for these calls."""
    _require(stage, "stage", torch.int32)
    _require(residual, "residual", torch.float32, 2)
    _require(counter, "counter", torch.int32)
    rows, h = residual.shape
    g, b = _affine(gamma, beta, h, residual.device)
    ib = _bias_vector(bias, h, torch.float32, residual.device)
    out = torch.empty_like(residual)
    arr = (_ptr * len(q_dst_ptrs))(*q_dst_ptrs)
    pads = (_ptr * len(pad_ptrs))(*pad_ptrs)
    with _on_device(residual.device):
        rc = _c_tp_exchange_reduce_ln_q(stage.data_ptr(), n_partials, partial_stride, float(scale), ib.data_ptr(),
                                        residual.data_ptr(), g.data_ptr(), b.data_ptr(), float(epsilon),
                                        out.data_ptr(), arr, len(q_dst_ptrs), q_row_offset, rows, h, pads, rank,
                                        len(pad_ptrs), epoch & 0xFFFFFFFF, counter.data_ptr(), int(limit_ms),
                                        _stream_ptr(residual.device))
    _check(rc)
    return out


def tp_barrier(pad_ptrs, rank, epoch, device, limit_ms=2000):
    """Stream-ordered barrier over the ranks owning the pads at pad_ptrs (ti_tp_barrier_limit); the wait
    gives up after limit_ms and sets the status word."""
    arr = (_ptr * len(pad_ptrs))(*pad_ptrs)
    with _on_device(device):
        rc = _c_tp_barrier(arr, rank, len(pad_ptrs), epoch & 0xFFFFFFFF, int(limit_ms), _stream_ptr(device))
    _check(rc)


def decode_attention(qkv, keys, values_t, position, alpha_qk, alpha_pv):
    """Attention of one new token per sequence over the int8 cache (ti_decode_attention_s8).
    qkv int8 [B(+pad), 3*E] (q | k | v of the token); keys [B, cap, E]; values_t [B, Hl, D, cap];
    position: int32 device tensor with the number of cached tokens.  Appends k and v to the cache
    and returns the int8 context [B, E]."""
    _require(keys, "keys", torch.int8, 3)
    _require(values_t, "values_t", torch.int8, 4)
    if not (isinstance(qkv, torch.Tensor) and qkv.is_cuda and qkv.dtype == torch.int8 and qkv.dim() == 2
            and qkv.stride(1) == 1):
        raise RuntimeError("qkv must be a 2-dimensional CUDA int8 tensor with contiguous rows")
    if not (isinstance(position, torch.Tensor) and position.is_cuda and position.dtype == torch.int32
            and position.numel() == 1):
        raise RuntimeError("position must be a CUDA int32 tensor with one element")
    b, hl, d, cap = values_t.shape
    e = hl * d
    if keys.shape != (b, cap, e) or qkv.shape[0] < b or qkv.shape[1] < 3 * e:
        raise RuntimeError(f"keys {tuple(keys.shape)}, values_t {tuple(values_t.shape)} and qkv {tuple(qkv.shape)} disagree")
    ctx = torch.empty((b, e), dtype=torch.int8, device=qkv.device)
    with _on_device(qkv.device):
        rc = _c_decode_attention(qkv.data_ptr(), qkv.stride(0), keys.data_ptr(), values_t.data_ptr(), b, hl, d, cap,
                                 position.data_ptr(), float(alpha_qk), float(alpha_pv), ctx.data_ptr(), e,
                                 _stream_ptr(qkv.device))
    _check(rc)
    return ctx


def attention_prefill(q, k_rows, vt, out, *, batch, heads, head_dim, tgt_len, src_len, ld_q, q_batch_stride,
                      ld_k, k_batch_stride, ld_vt, alpha_qk, alpha_pv):
    """Causal prefill attention in one kernel (ti_attention_prefill_s8): int8 views q (query rows, row
    stride ld_q, head h at column h*head_dim), k_rows (key rows) and vt ([batch, heads, head_dim, ld_vt],
    keys contiguous) -> int8 context written into out [batch, tgt_len, heads*head_dim].  Row t sees keys
    j <= t + (src_len - tgt_len)."""
    for t, name in ((q, "q"), (k_rows, "k_rows"), (vt, "vt"), (out, "out")):
        if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.int8):
            raise RuntimeError(f"{name} must be a CUDA int8 tensor")
    el = heads * head_dim
    if out.shape != (batch, tgt_len, el) or not out.is_contiguous():
        raise RuntimeError(f"out must be a contiguous [{batch}, {tgt_len}, {el}] tensor, got {tuple(out.shape)}")
    with _on_device(q.device):
        rc = _c_attention_prefill(q.data_ptr(), ld_q, q_batch_stride, k_rows.data_ptr(), ld_k, k_batch_stride,
                                  vt.data_ptr(), ld_vt, out.data_ptr(), el, tgt_len * el, batch, heads, head_dim,
                                  tgt_len, src_len, float(alpha_qk), float(alpha_pv), _stream_ptr(q.device))
    _check(rc)
    return out


def advance_position(position, by=1):
    """position += by on the current stream (ti_advance_position)."""
    with _on_device(position.device):
        rc = _c_advance_position(position.data_ptr(), int(by), _stream_ptr(position.device))
    _check(rc)


def transpose_values(v, vt, col0=0):
    """int8 v [B, T, H, D] -> vt [B, H, D, cap] at columns [col0, col0 + T): the transposed
    value layout P.V consumes.  Replaces transpose(1, 2).contiguous() of torch_int/models/opt.py:180."""
    _require(vt, "vt", torch.int8, 4)
    if not (isinstance(v, torch.Tensor) and v.is_cuda and v.dtype == torch.int8 and v.dim() == 4):
        raise RuntimeError("v must be a 4-dimensional CUDA int8 tensor")
    b, t, h, d = v.shape
    # v may be a column block of a wider projection output: heads and head_dim contiguous,
    # tokens `ld_in` apart, sequences t * ld_in apart
    ld_in = v.stride(1)
    if v.stride(3) != 1 or v.stride(2) != d or (b > 1 and v.stride(0) != t * ld_in):
        raise RuntimeError(f"v has unsupported strides {v.stride()} for shape {tuple(v.shape)}")
    if vt.shape[:3] != (b, h, d) or vt.shape[3] < col0 + t or vt.device != v.device:
        raise RuntimeError(f"vt {tuple(vt.shape)} cannot hold v {tuple(v.shape)} at column {col0}")
    with _on_device(v.device):
        rc = _c_transpose_values(v.data_ptr(), vt.data_ptr(), b, t, h, d, ld_in, vt.shape[3], col0,
                                 _stream_ptr(v.device))
    _check(rc)
    return vt


def set_dependent_launch(on):
    """Programmatic dependent launch of the small-M GEMMs on (default) or off; see ti_set_dependent_launch."""
    _c_set_dependent_launch(1 if on else 0)


def set_narrow_a(on):
    """16-row A stages for GEMMs of at most 16 rows on (default) or off; see ti_set_narrow_a."""
    _c_set_narrow_a(1 if on else 0)


def set_group_m(tiles):
    """Tuning knob: M tiles per band of the GEMM tile order (0 = automatic); see ti_set_group_m."""
    _c_set_group_m(int(tiles))


def set_sm_limit(sms):
    """Caps the SMs the persistent GEMM grids occupy (0 = all); see ti_set_sm_limit."""
    _c_set_sm_limit(int(sms))


def device_status(reset=True):
    """Synchronises the current device and returns the kernels' status word
    (0 = ok; otherwise the code of the first in-kernel wait that timed out).
    With reset, a non-zero word is cleared and so is the split-K scratch of the current device (a
    launch that gave up may have left partial sums and counters in it, and every later small-M
    GEMM expects it all zero)."""
    v = ctypes.c_int(0)
    _check(_c_device_status(ctypes.byref(v), 1 if reset else 0))
    if reset and v.value != 0:
        ws = _workspaces.get(torch.cuda.current_device())
        if ws is not None:
            ws.zero_()
            torch.cuda.synchronize(ws.device)
    return v.value
