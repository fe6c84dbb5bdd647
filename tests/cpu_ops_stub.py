"""CPU stand-ins for the functions of torch_int._CUDA, evaluated with the oracle.

TEST INFRASTRUCTURE ONLY.  The product has no CPU path: torch_int._CUDA raises on CPU tensors.  These
stand-ins exist so that the HOST logic of torch_int.models (strides and views handed to the strided GEMM,
cache bookkeeping, masks, the order of the fused residual/LayerNorm steps, decoding) can be exercised in
the CPU test-suite: a test monkeypatches the module attribute `C` of torch_int.models.opt / kv_cache (and
the op names imported by torch_int.nn.*) with this module and compares the model's output with the
oracle's restatement of the reference model.  Every function has the signature of its namesake in
torch_int/_CUDA.py; nothing here is imported by the package.
"""
import numpy as np
import torch

from oracle import w8a8 as O

EPI_S8_BIAS_S8, EPI_S8_BIAS_S8_RELU, EPI_F32_BIAS_F32, EPI_S32_BIAS_S32_ADD, \
    EPI_S32_BIAS_S32_SCALE, EPI_F32_ALPHA, EPI_S8_ALPHA, EPI_S32_RAW, EPI_S8_BIAS_S8_VEC, \
    EPI_F32_BIAS_F32_ACC = range(10)
_KIND = {EPI_S8_BIAS_S8: "b8_o8", EPI_S8_BIAS_S8_RELU: "relu_b8_o8", EPI_F32_BIAS_F32: "bfp32_ofp32",
         EPI_S32_BIAS_S32_ADD: "b32_o32", EPI_S32_BIAS_S32_SCALE: "b32_o32_with_scaling",
         EPI_F32_ALPHA: "f32t", EPI_S8_ALPHA: "s8t", EPI_S32_RAW: "s32t"}

launch_count = 0


def _acc(a2d, b2d):
    return O.gemm_acc(a2d.contiguous(), b2d.contiguous())


# ----------------------------------------------------------------------------- the reference's nine ops
linear_a8_w8_b8_o8 = O.linear_a8_w8_b8_o8
linear_relu_a8_w8_b8_o8 = O.linear_relu_a8_w8_b8_o8
linear_a8_w8_bfp32_ofp32 = O.linear_a8_w8_bfp32_ofp32
linear_a8_w8_b32_o32 = O.linear_a8_w8_b32_o32
linear_a8_w8_b32_o32_with_scaling = O.linear_a8_w8_b32_o32_with_scaling
bmm_s8t_s8n_s8t = O.bmm_s8t_s8n_s8t
bmm_s8t_s8n_f32t = O.bmm_s8t_s8n_f32t
bmm_s8t_s8n_s32t = O.bmm_s8t_s8n_s32t
dq_add_layernorm_q = O.dq_add_layernorm_q


def layernorm_q(x, gamma, beta, epsilon, fp32_norm=True):
    return O.layernorm_q(x, gamma if fp32_norm else gamma.to(x.dtype), beta if fp32_norm else beta.to(x.dtype), epsilon)


def dq_add_layernorm_q_bias(input, input_scale, input_bias, residual_input, gamma, beta, epsilon):
    if input_bias is None:
        return O.dq_add_layernorm_q(input, input_scale, residual_input, gamma, beta, epsilon)
    return O.dq_add_layernorm_q_bias(input, input_scale, input_bias.reshape(-1), residual_input, gamma, beta, epsilon)


# ----------------------------------------------------------------------------- extras
def gemm_i8_ex(a, b, out, bias=None, *, epilogue, m, n, k, batch=1, batch2=1, lda, ldb, ldc,
               stride_a=0, stride_b=0, stride_c=0, stride2_a=0, stride2_b=0, stride2_c=0,
               alpha=1.0, beta=0.0, tile_n=0, cta_pair=0, scatter_ptrs=None, scatter_rows=0,
               alpha_vec=None, beta_vec=None, splits=0):
    assert not scatter_rows, "the row-block scatter has no CPU stand-in"
    av = a.as_strided((batch2, batch, m, k), (stride2_a, stride_a, lda, 1))
    bv = b.as_strided((batch2, batch, n, k), (stride2_b, stride_b, ldb, 1))
    cv = out.as_strided((batch2, batch, m, n), (stride2_c, stride_c, ldc, 1))
    for i2 in range(batch2):
        for i1 in range(batch):
            acc = _acc(av[i2, i1], bv[i2, i1])
            if epilogue == EPI_S8_BIAS_S8_VEC:
                f = acc.numpy().astype(np.float32)
                t = (beta_vec.numpy().astype(np.float32) * bias.reshape(-1).numpy().astype(np.float32)).astype(np.float32)
                y = (alpha_vec.numpy().astype(np.float64)[None, :] * f.astype(np.float64) +
                     t.astype(np.float64)[None, :]).astype(np.float32)
                res = torch.from_numpy(np.clip(np.rint(y.astype(np.float64)), -128, 127).astype(np.int8))
            elif epilogue == EPI_F32_BIAS_F32_ACC:  # the fp32 linear's output added to what C holds
                res = cv[i2, i1] + O.epilogue_numpy(acc, bias, alpha, beta, "bfp32_ofp32")
            else:
                res = O.epilogue_numpy(acc, bias, alpha, beta, _KIND[epilogue])
            cv[i2, i1].copy_(res)
    return out


def softmax_q(scores, mask=None, num_heads=1, causal=-1):
    bh, t, s = scores.shape
    if mask is None and causal >= 0:
        cols = torch.arange(s).view(1, s)
        rows = torch.arange(t).view(t, 1) + causal
        m = torch.zeros((t, s), dtype=torch.float32)
        m[cols > rows] = torch.finfo(torch.float32).min
        mask = m.view(1, 1, t, s).expand(bh // num_heads, 1, t, s).contiguous()
    elif mask is not None:
        mask = mask.reshape(bh // num_heads, 1, t, s)
    return O.softmax_q(scores, mask)


def transpose_values(v, vt, col0=0):
    b, t, h, d = v.shape
    vt[:, :, :, col0:col0 + t] = v.permute(0, 2, 3, 1)
    return vt


def _attend(q, k, vt, alpha_qk, alpha_pv, past):
    """q [T,D], k [S,D], vt [D,S] of one head -> int8 [T,D]; row t sees keys j <= t + past."""
    t, s = q.shape[0], k.shape[0]
    scores = O.bmm_s8t_s8n_f32t(q.reshape(1, t, -1).contiguous(), k.reshape(1, s, -1).contiguous(), alpha_qk)
    probs = softmax_q(scores, None, 1, causal=past)
    return O.bmm_s8t_s8n_s8t(probs, vt.reshape(1, -1, s).contiguous(), alpha_pv)[0]


def attention_prefill(q, k_rows, vt, out, *, batch, heads, head_dim, tgt_len, src_len, ld_q, q_batch_stride,
                      ld_k, k_batch_stride, ld_vt, alpha_qk, alpha_pv):
    d = head_dim
    qv = q.as_strided((batch, heads, tgt_len, d), (q_batch_stride, d, ld_q, 1))
    kv = k_rows.as_strided((batch, heads, src_len, d), (k_batch_stride, d, ld_k, 1))
    vv = vt.as_strided((batch, heads, d, src_len), (heads * d * ld_vt, d * ld_vt, ld_vt, 1))
    ov = out.view(batch, tgt_len, heads, d)
    for b in range(batch):
        for h in range(heads):
            ov[b, :, h] = _attend(qv[b, h], kv[b, h], vv[b, h], alpha_qk, alpha_pv, src_len - tgt_len)
    return out


def decode_attention(qkv, keys, values_t, position, alpha_qk, alpha_pv):
    b, hl, d, cap = values_t.shape
    e = hl * d
    pos = int(position.item())
    assert 0 <= pos < cap
    ctx = torch.empty((b, e), dtype=torch.int8)
    keys[:, pos] = qkv[:b, e:2 * e]
    values_t[:, :, :, pos] = qkv[:b, 2 * e:3 * e].view(b, hl, d)
    for i in range(b):
        for h in range(hl):
            q = qkv[i, h * d:(h + 1) * d].view(1, d)
            ctx[i, h * d:(h + 1) * d] = _attend(q, keys[i, :pos + 1, h * d:(h + 1) * d],
                                               values_t[i, h, :, :pos + 1], alpha_qk, alpha_pv, pos)[0]
    return ctx


def advance_position(position, by=1):
    position += by


def device_status(reset=False):
    return 0


# ----------------------------------------------------------------------------- installation
def install(setattr_fn=setattr):
    """Puts this module in place of torch_int._CUDA inside torch_int.models / torch_int.nn.  `setattr_fn`
    is monkeypatch.setattr in a pytest process (undone at teardown) or plain setattr in a child process."""
    import sys
    import torch_int.models.kv_cache as kv_mod
    import torch_int.models.opt as opt_mod
    import torch_int.nn.bmm as bmm_mod
    import torch_int.nn.fused as fused_mod
    import torch_int.nn.linear as linear_mod
    this = sys.modules[__name__]
    setattr_fn(opt_mod, "C", this)
    setattr_fn(kv_mod, "C", this)
    for mod in (linear_mod, bmm_mod, fused_mod):
        for name in dir(this):
            if not name.startswith("_") and callable(getattr(this, name)) and hasattr(mod, name):
                setattr_fn(mod, name, getattr(this, name))


class _NoStream:
    """Stand-in for torch.cuda.Stream / Event on CPU ranks: everything runs in program order."""

    def __init__(self, *args, **kwargs):
        pass

    def record(self, stream=None):
        pass

    def wait_event(self, event):
        pass

    def wait_stream(self, stream):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def install_serial_streams(setattr_fn=setattr):
    """torch.cuda streams and events become no-ops (CPU ranks run the pipelined layer loop in program order)."""
    setattr_fn(torch.cuda, "current_stream", lambda device=None: _NoStream())
    setattr_fn(torch.cuda, "Stream", _NoStream)
    setattr_fn(torch.cuda, "Event", _NoStream)
    setattr_fn(torch.cuda, "stream", lambda s: _NoStream())
    setattr_fn(torch.Tensor, "record_stream", lambda self, stream: None)
