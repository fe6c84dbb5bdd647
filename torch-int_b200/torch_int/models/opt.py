"""Int8 OPT: attention, decoder layer, decoder, model and causal LM built on the
W8A8 operators.  Class names, constructor arguments, sub-module and buffer
names and the ``from_float`` conversions follow torch_int/models/opt.py, so a
state dict exported for the reference loads here.

Two ways to run a layer:

* ``forward`` of ``Int8OPTAttention`` / ``Int8OPTDecoderLayer`` keeps the
  reference call signatures and return tuples (opt.py:83-199, 244-299),
  including the ``(key, value)`` int8 tuples of shape [B, H, S, D] as cache.
* the decoder itself drives the layers through ``forward_fused``: q/k/v are
  multiplied as strided views (no head-transposing copies, opt.py:80-81,191-196),
  the mask/softmax/x127/round chain is one kernel, keys and transposed values
  live in a pre-allocated int8 cache (no ``torch.cat``, opt.py:113-116,180), and
  the two residual updates are fused with the following LayerNorm-quantise
  (int32 GEMM output -> ``dq_add_layernorm_q`` with the linear's fp32 bias).
  With fp32 activations this wiring performs exactly the reference's fp32
  operations: d = fma(alpha, acc, bias), residual + d, LayerNorm, quantise.

Unlike the reference, nothing here inherits from ``transformers``: the
reference borrows ``OPTDecoder.forward`` and the mask helper of the
transformers release it was written against (opt.py:346-349,407-410,442-450),
which later releases no longer provide.  The embedding, position, mask and
final LayerNorm logic of OPT is therefore restated in ``Int8OPTDecoder.forward``.
``from_float`` still accepts the float ``transformers`` OPT modules.

Tensor parallelism: pass a ``TensorParallel`` context (models/tensor_parallel.py);
q/k/v/fc1 are sharded by output features (whole heads per rank), out_proj/fc2 by
input features, and the int32 partial sums of the latter two are all-reduced
before the fused residual/LayerNorm kernel, so every rank count gives
bit-identical results.
"""
import math
import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
from torch import nn

from .. import _CUDA as C
from ..nn.bmm import BMM_S8T_S8N_F32T, BMM_S8T_S8N_S8T
from ..nn.fused import LayerNormQ
from ..nn.linear import W8A8B8O8Linear, W8A8B8O8LinearReLU, W8A8BFP32OFP32Linear
from .kv_cache import StaticInt8KVCache
from .tensor_parallel import TensorParallel


@dataclass
class Int8OPTConfig:
    """The fields of transformers' OPTConfig that the Int8 OPT classes read."""
    vocab_size: int = 50272
    hidden_size: int = 768
    num_hidden_layers: int = 12
    ffn_dim: int = 3072
    num_attention_heads: int = 12
    max_position_embeddings: int = 2048
    word_embed_proj_dim: Optional[int] = None
    pad_token_id: int = 1
    do_layer_norm_before: bool = True
    _remove_final_layer_norm: bool = False

    def __post_init__(self):
        if self.word_embed_proj_dim is None:
            self.word_embed_proj_dim = self.hidden_size


# TI_TP_CHECK_EVERY_PASS=1: read the kernels' status word (a device synchronisation and one small
# collective) after EVERY tensor-parallel forward pass, not only after the first one of a workspace.
_CHECK_EVERY_PASS = os.environ.get("TI_TP_CHECK_EVERY_PASS", "0") == "1"
_RESIDUAL_IN_GEMM_MIN_ROWS = 128  # below this the GEMMs split K and reduce in scratch: the row kernel keeps the add


def _round_up(v, m):
    return (v + m - 1) // m * m


class Int8OPTAttention(nn.Module):
    """Multi-head self-attention on int8 activations (opt.py:22-199)."""

    def __init__(self, embed_dim: int, num_heads: int, tp: Optional[TensorParallel] = None):
        super().__init__()
        self.embed_dim = embed_dim
        self.num_heads = num_heads
        self.head_dim = embed_dim // num_heads
        if self.head_dim * num_heads != embed_dim:
            raise ValueError(f"embed_dim must be divisible by num_heads (got `embed_dim`: {embed_dim}"
                             f" and `num_heads`: {num_heads}).")
        self.tp = tp if tp is not None else TensorParallel.single()
        if num_heads % self.tp.size != 0:
            raise ValueError(f"{num_heads} heads cannot be split over {self.tp.size} ranks")
        self.local_heads = num_heads // self.tp.size
        self.local_dim = self.local_heads * self.head_dim
        self.attention_weight_scale = 1.0
        # Causal, padding-free attention with head_dim 64 or 128 runs as one fused kernel
        # (C.attention_prefill); everything else, and all inputs when this is False
        # (TI_FUSED_ATTENTION=0), goes through scores GEMM -> softmax_q -> context GEMM.  The two forms
        # agree except where a probability sits on a rounding tie (the row sum is accumulated in a
        # different order), which can move a context value by one unit.
        self.fused_attention = os.environ.get("TI_FUSED_ATTENTION", "1") != "0"
        self.qk_bmm = BMM_S8T_S8N_F32T(1.0)
        self.pv_bmm = BMM_S8T_S8N_S8T(1.0)
        # column-parallel: each rank owns whole heads
        self.k_proj = W8A8B8O8Linear(embed_dim, self.local_dim)
        self.v_proj = W8A8B8O8Linear(embed_dim, self.local_dim)
        self.q_proj = W8A8B8O8Linear(embed_dim, self.local_dim)
        # row-parallel: each rank owns a slice of the input features
        self.out_proj = W8A8BFP32OFP32Linear(self.local_dim, embed_dim)

    @staticmethod
    @torch.no_grad()
    def from_float(module, input_scale: float, q_output_scale: float, k_output_scale: float,
                   v_output_scale: float, out_input_scale: float):
        """Quantises a float OPTAttention (opt.py:53-78).  The 1/sqrt(d) scaling is
        folded into q_proj; the float module is left untouched."""
        int8_module = Int8OPTAttention(module.embed_dim, module.num_heads)
        scaling = module.scaling
        q_output_scale = q_output_scale * scaling
        q_float = nn.Linear(module.embed_dim, module.embed_dim)
        q_float.weight = nn.Parameter(module.q_proj.weight.detach() * scaling)
        q_float.bias = nn.Parameter(module.q_proj.bias.detach() * scaling)
        int8_module.q_proj = W8A8B8O8Linear.from_float(q_float, input_scale, q_output_scale)
        int8_module.k_proj = W8A8B8O8Linear.from_float(module.k_proj, input_scale, k_output_scale)
        int8_module.v_proj = W8A8B8O8Linear.from_float(module.v_proj, input_scale, v_output_scale)
        int8_module.out_proj = W8A8BFP32OFP32Linear.from_float(module.out_proj, out_input_scale)
        int8_module.qk_bmm = BMM_S8T_S8N_F32T.from_scale(q_output_scale, k_output_scale)
        # alpha = s_prob * s_v / s_out with s_prob = 1/127
        int8_module.pv_bmm = BMM_S8T_S8N_S8T.from_scale(1.0 / 127, v_output_scale, out_input_scale)
        return int8_module

    def _fused_qkv(self):
        """Concatenated [3*El, E] weight, [3*El] bias and per-column alpha / beta vectors of the
        q, k and v projections, for running them as one GEMM.  Built on first use; the three
        modules' weight buffers are then re-pointed at row blocks of the concatenated tensor, so
        no second copy of the weights is kept.  Rebuilt if a buffer is replaced or modified."""
        mods = (self.q_proj, self.k_proj, self.v_proj)
        key = tuple((m.weight.data_ptr(), m.weight._version, m.bias.data_ptr(), m.bias._version,
                     m._scalar("a"), m._scalar("b")) for m in mods)
        hit = getattr(self, "_qkv_cache", None)
        if hit is not None and hit[0] == key:
            return hit[1]
        el = self.local_dim
        dev = self.q_proj.weight.device
        w = torch.cat([m.weight for m in mods], dim=0).contiguous()
        bias = torch.cat([m.bias.reshape(-1) for m in mods], dim=0).contiguous()
        alpha = torch.cat([torch.full((el,), m._scalar("a"), dtype=torch.float32, device=dev) for m in mods])
        beta = torch.cat([torch.full((el,), m._scalar("b"), dtype=torch.float32, device=dev) for m in mods])
        for i, m in enumerate(mods):
            m.weight = w[i * el:(i + 1) * el]
            m.bias = bias[i * el:(i + 1) * el].view(1, el)
        key = tuple((m.weight.data_ptr(), m.weight._version, m.bias.data_ptr(), m.bias._version,
                     m._scalar("a"), m._scalar("b")) for m in mods)
        object.__setattr__(self, "_qkv_cache", (key, (w, bias, alpha, beta)))
        return w, bias, alpha, beta

    def _shape(self, tensor: torch.Tensor, seq_len: int, bsz: int):
        return tensor.view(bsz, seq_len, self.local_heads, self.head_dim).transpose(1, 2).contiguous()

    # ------------------------------------------------------------------ fast path
    def attention_core(self, q, q_row_stride, k_rows, vt, bsz, tgt_len, src_len, src_pad, k_row_stride,
                       k_batch_stride, vt_row_stride, causal, mask):
        """softmax(q k^T) v on strided views.  q: query rows [B*T, Hl*D] with row stride
        `q_row_stride`; k_rows: key rows with row stride `k_row_stride` and batch stride
        `k_batch_stride`; vt: transposed values [B,Hl,D,*] with row stride `vt_row_stride`.
        Returns int8 [B,T,Hl*D]."""
        hl, d, el = self.local_heads, self.head_dim, self.local_dim
        dev = q.device
        if self.fused_attention and mask is None and causal >= 0 and d in (64, 128):
            # one kernel; scores and probabilities stay on the SM
            out = torch.empty((bsz, tgt_len, el), dtype=torch.int8, device=dev)
            return C.attention_prefill(q, k_rows, vt, out, batch=bsz, heads=hl, head_dim=d, tgt_len=tgt_len,
                                       src_len=src_len, ld_q=q_row_stride, q_batch_stride=tgt_len * q_row_stride,
                                       ld_k=k_row_stride, k_batch_stride=k_batch_stride, ld_vt=vt_row_stride,
                                       alpha_qk=self.qk_bmm._alpha(), alpha_pv=self.pv_bmm._alpha())
        scores = torch.empty((bsz * hl, tgt_len, src_pad), dtype=torch.float32, device=dev)
        C.gemm_i8_ex(q, k_rows, scores, epilogue=C.EPI_F32_ALPHA, m=tgt_len, n=src_pad, k=d,
                     batch=hl, batch2=bsz, lda=q_row_stride, ldb=k_row_stride, ldc=src_pad,
                     stride_a=d, stride_b=d, stride_c=tgt_len * src_pad,
                     stride2_a=tgt_len * q_row_stride, stride2_b=k_batch_stride, stride2_c=hl * tgt_len * src_pad,
                     alpha=self.qk_bmm._alpha())
        probs = C.softmax_q(scores, mask, hl, causal=causal)
        del scores
        out = torch.empty((bsz, tgt_len, el), dtype=torch.int8, device=dev)
        C.gemm_i8_ex(probs, vt, out, epilogue=C.EPI_S8_ALPHA, m=tgt_len, n=d, k=src_pad,
                     batch=hl, batch2=bsz, lda=src_pad, ldb=vt_row_stride, ldc=el,
                     stride_a=tgt_len * src_pad, stride_b=d * vt_row_stride, stride_c=d,
                     stride2_a=hl * tgt_len * src_pad, stride2_b=hl * d * vt_row_stride,
                     stride2_c=tgt_len * el, alpha=self.pv_bmm._alpha())
        return out

    @torch.no_grad()
    def forward_fused(self, hidden_int8, cache: Optional[StaticInt8KVCache], layer_idx: int, past_len: int,
                      mask: Optional[torch.Tensor], out: Optional[torch.Tensor] = None, b0: int = 0,
                      context_only: bool = False, decode: bool = False):
        """int8 [B,T,E] -> int32 partial sums of out_proj [B*T, E] (this rank's input
        slice; bias and scale are applied after the reduction over the ranks).  `out`:
        optional destination; `b0`: index of the first of these sequences in the cache."""
        bsz, tgt_len, _ = hidden_int8.shape
        hl, d, el = self.local_heads, self.head_dim, self.local_dim
        x2d = hidden_int8.view(-1, self.embed_dim)
        tokens = x2d.shape[0]
        src_len = (past_len or 0) + tgt_len
        src_pad = _round_up(src_len, 16)
        # q, k and v in ONE GEMM over the concatenated weights (per-column alpha / beta); 16 spare
        # rows at the end keep the padded key reads of the last sequence inside the allocation
        w, bias, alpha_vec, beta_vec = self._fused_qkv()
        qkv = torch.empty((tokens + 16, 3 * el), dtype=torch.int8, device=x2d.device)
        C.gemm_i8_ex(x2d, w, qkv, bias, epilogue=C.EPI_S8_BIAS_S8_VEC, m=tokens, n=3 * el, k=self.embed_dim,
                     lda=self.embed_dim, ldb=self.embed_dim, ldc=3 * el, alpha_vec=alpha_vec, beta_vec=beta_vec)
        ld = 3 * el
        if decode:
            # one new token per sequence: append + scores + softmax + context in one kernel that reads
            # the position from device memory (no per-step host parameters: CUDA-graph friendly)
            ctx = C.decode_attention(qkv, cache.keys[layer_idx][b0:b0 + bsz], cache.values_t[layer_idx][b0:b0 + bsz],
                                     cache.pos, self.qk_bmm._alpha(), self.pv_bmm._alpha()).view(bsz, 1, el)
            if context_only:
                return ctx
            acc = out if out is not None else torch.empty((bsz, self.embed_dim), dtype=torch.int32, device=ctx.device)
            C.gemm_i8_ex(ctx.view(bsz, el), self.out_proj.weight, acc, epilogue=C.EPI_S32_RAW, m=bsz,
                         n=self.embed_dim, k=el, lda=el, ldb=el, ldc=self.embed_dim)
            return acc
        q = qkv[:tokens, :el]
        k3 = qkv[:tokens].view(bsz, tgt_len, ld)[:, :, el:2 * el]
        v3 = qkv[:tokens].view(bsz, tgt_len, ld)[:, :, 2 * el:]
        if cache is not None:
            k_rows, vt = cache.store(layer_idx, k3, v3, bsz, tgt_len, past_len, b0)
            k_row_stride, k_batch_stride, vt_row_stride = el, cache.capacity * el, cache.capacity
        else:
            # keys are read in place; rows [T, src_pad) of a sequence are the first rows of the next one
            # (or the spare rows): finite garbage that the causal limit masks
            k_rows, k_row_stride, k_batch_stride = qkv[:, el:2 * el], ld, tgt_len * ld
            vt = (torch.zeros if src_pad != src_len else torch.empty)((bsz, hl, d, src_pad), dtype=torch.int8,
                                                                      device=x2d.device)
            C.transpose_values(v3.as_strided((bsz, tgt_len, hl, d), (tgt_len * ld, ld, d, 1)), vt, 0)
            vt_row_stride = src_pad
        causal = past_len if mask is None else -1
        ctx = self.attention_core(q, ld, k_rows, vt, bsz, tgt_len, src_len, src_pad,
                                  k_row_stride, k_batch_stride, vt_row_stride, causal, mask)
        if context_only:
            return ctx  # int8 [B,T,Hl*D]: the caller runs out_proj itself
        ctx2d = ctx.view(-1, el)
        acc = out if out is not None else torch.empty((ctx2d.shape[0], self.embed_dim), dtype=torch.int32,
                                                      device=ctx.device)
        C.gemm_i8_ex(ctx2d, self.out_proj.weight, acc, epilogue=C.EPI_S32_RAW, m=ctx2d.shape[0],
                     n=self.embed_dim, k=el, lda=el, ldb=el, ldc=self.embed_dim)
        return acc

    # ------------------------------------------------------- reference signature
    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor, key_value_states: Optional[torch.Tensor] = None,
                past_key_value: Optional[Tuple[torch.Tensor]] = None,
                attention_mask: Optional[torch.Tensor] = None,
                layer_head_mask: Optional[torch.Tensor] = None, output_attentions: bool = False
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[Tuple[torch.Tensor]]]:
        """Input shape: Batch x Time x Channel (int8).  Returns (attn_output fp32,
        attention probabilities or None, (key_states, value_states) int8 [B,H,S,D])."""
        if self.tp.size != 1:
            raise RuntimeError("the reference-signature forward is single-GPU; the decoder uses forward_fused")
        is_cross_attention = key_value_states is not None
        bsz, tgt_len, _ = hidden_states.size()
        query_states = self.q_proj(hidden_states)
        if is_cross_attention and past_key_value is not None:
            key_states, value_states = past_key_value[0], past_key_value[1]
        elif is_cross_attention:
            key_states = self._shape(self.k_proj(key_value_states), -1, bsz)
            value_states = self._shape(self.v_proj(key_value_states), -1, bsz)
        elif past_key_value is not None:
            key_states = self._shape(self.k_proj(hidden_states), -1, bsz)
            value_states = self._shape(self.v_proj(hidden_states), -1, bsz)
            key_states = torch.cat([past_key_value[0], key_states], dim=2)
            value_states = torch.cat([past_key_value[1], value_states], dim=2)
        else:
            key_states = self._shape(self.k_proj(hidden_states), -1, bsz)
            value_states = self._shape(self.v_proj(hidden_states), -1, bsz)
        past_key_value = (key_states, value_states)

        proj_shape = (bsz * self.num_heads, -1, self.head_dim)
        query_states = self._shape(query_states, tgt_len, bsz).view(*proj_shape)
        key_states = key_states.reshape(*proj_shape)
        value_states = value_states.reshape(*proj_shape)
        src_len = key_states.size(1)
        if src_len % 16 != 0:
            raise RuntimeError(f"the key length ({src_len}) must be a multiple of 16 in the reference-signature "
                               "forward (the reference pads sequences for the same reason, opt.py:375-383)")
        if attention_mask is not None and attention_mask.size() != (bsz, 1, tgt_len, src_len):
            raise ValueError(f"Attention mask should be of size {(bsz, 1, tgt_len, src_len)}, "
                             f"but is {attention_mask.size()}")
        attn_weights = self.qk_bmm(query_states, key_states)
        attn_probs_reshaped = None
        if layer_head_mask is None and not output_attentions:
            mask = None if attention_mask is None else attention_mask.to(torch.float32).contiguous()
            attn_probs = C.softmax_q(attn_weights, mask, self.num_heads)
        else:
            # rarely used options: follow the reference's torch formulation (opt.py:139-178)
            if attention_mask is not None:
                attn_weights = attn_weights.view(bsz, self.num_heads, tgt_len, src_len) + attention_mask
                attn_weights = torch.max(attn_weights, torch.tensor(torch.finfo(attn_weights.dtype).min,
                                                                    device=attn_weights.device))
                attn_weights = attn_weights.view(bsz * self.num_heads, tgt_len, src_len)
            attn_probs = nn.functional.softmax(attn_weights, dim=-1)
            if layer_head_mask is not None:
                if layer_head_mask.size() != (self.num_heads,):
                    raise ValueError(f"Head mask for a single layer should be of size {(self.num_heads,)}, "
                                     f"but is {layer_head_mask.size()}")
                attn_probs = layer_head_mask.view(1, -1, 1, 1) * attn_probs.view(bsz, self.num_heads, tgt_len, src_len)
                attn_probs = attn_probs.view(bsz * self.num_heads, tgt_len, src_len)
            if output_attentions:
                attn_probs_reshaped = attn_probs.view(bsz, self.num_heads, tgt_len, src_len).clone()
            attn_probs = attn_probs.mul(127).round().to(torch.int8)
        value_states = value_states.transpose(1, 2).contiguous()
        attn_output = self.pv_bmm(attn_probs, value_states)
        attn_output = attn_output.view(bsz, self.num_heads, tgt_len, self.head_dim).transpose(1, 2)
        attn_output = attn_output.reshape(bsz, tgt_len, self.embed_dim).contiguous()
        attn_output = self.out_proj(attn_output)
        return attn_output, attn_probs_reshaped, past_key_value


class Int8OPTDecoderLayer(nn.Module):
    """Pre-LayerNorm OPT decoder layer on the W8A8 operators (opt.py:202-299)."""

    def __init__(self, embed_dim, num_attention_heads, ffn_dim, tp: Optional[TensorParallel] = None):
        super().__init__()
        self.embed_dim = embed_dim
        self.tp = tp if tp is not None else TensorParallel.single()
        if ffn_dim % self.tp.size != 0:
            raise ValueError(f"ffn_dim {ffn_dim} cannot be split over {self.tp.size} ranks")
        self.local_ffn = ffn_dim // self.tp.size
        self.self_attn = Int8OPTAttention(embed_dim=embed_dim, num_heads=num_attention_heads, tp=self.tp)
        self.self_attn_layer_norm = LayerNormQ(embed_dim)
        self.fc1 = W8A8B8O8LinearReLU(embed_dim, self.local_ffn)       # column-parallel
        self.fc2 = W8A8BFP32OFP32Linear(self.local_ffn, embed_dim)     # row-parallel
        # Prefill on one GPU: out_proj and fc2 add their output to the fp32 residual in the GEMM epilogue
        # (TI_RESIDUAL_IN_GEMM=0: the int32 products go through the fused residual/LayerNorm row kernel
        # instead; same results bit for bit)
        self.residual_in_gemm = os.environ.get("TI_RESIDUAL_IN_GEMM", "1") != "0"
        self.final_layer_norm = LayerNormQ(embed_dim)

    @staticmethod
    def from_float(module, attn_input_scale: float, q_output_scale: float, k_output_scale: float,
                   v_output_scale: float, out_input_scale: float, fc1_input_scale: float,
                   fc2_input_scale: float):
        """Quantises a float OPTDecoderLayer with calibrated activation scales (opt.py:219-242)."""
        int8_module = Int8OPTDecoderLayer(module.embed_dim, module.self_attn.num_heads, module.fc1.out_features)
        int8_module.self_attn_layer_norm = LayerNormQ.from_float(module.self_attn_layer_norm, attn_input_scale)
        int8_module.self_attn = Int8OPTAttention.from_float(
            module.self_attn, attn_input_scale, q_output_scale, k_output_scale, v_output_scale, out_input_scale)
        int8_module.final_layer_norm = LayerNormQ.from_float(module.final_layer_norm, fc1_input_scale)
        int8_module.fc1 = W8A8B8O8LinearReLU.from_float(module.fc1, fc1_input_scale, fc2_input_scale)
        int8_module.fc2 = W8A8BFP32OFP32Linear.from_float(module.fc2, fc2_input_scale)
        return int8_module

    # ------------------------------------------------------------------ fast path
    @torch.no_grad()
    def forward_fused(self, residual, hidden_int8, cache, layer_idx, past_len, mask, next_ln: Optional[LayerNormQ],
                      decode: bool = False, inplace: bool = False):
        """residual fp [B,T,E], hidden_int8 = LayerNormQ(residual) -> (new residual,
        int8 input of the next layer or None).  `next_ln` is the next layer's
        self_attn_layer_norm (None after the last layer).  `inplace`: the caller owns `residual` and lets
        it be updated in place, as the reference's layer does (opt.py:281,289)."""
        shape = residual.shape
        attn = self.self_attn
        if (inplace and self.residual_in_gemm and not decode and self.tp.size == 1 and residual.dtype == torch.float32
                and residual.is_contiguous() and residual.numel() // self.embed_dim > _RESIDUAL_IN_GEMM_MIN_ROWS):
            # Prefill on one GPU with an fp32 residual stream: out_proj and fc2 add fma(a, acc, bias) to the
            # residual in their epilogues (same arithmetic as the fused row kernel below), and the row kernel
            # only normalises and quantises: the int32 products never travel through HBM.
            e = self.embed_dim
            res2d = residual.view(-1, e)
            ctx = attn.forward_fused(hidden_int8, cache, layer_idx, past_len, mask, context_only=True)
            ctx2d = ctx.view(-1, attn.local_dim)
            C.gemm_i8_ex(ctx2d, attn.out_proj.weight, res2d, attn.out_proj.bias, epilogue=C.EPI_F32_BIAS_F32_ACC,
                         m=res2d.shape[0], n=e, k=attn.local_dim, lda=attn.local_dim, ldb=attn.local_dim, ldc=e,
                         alpha=attn.out_proj._scalar("a"), beta=1.0)
            ln = self.final_layer_norm
            h8 = self.fc1._op(C.layernorm_q(res2d, ln.weight, ln.bias, ln.eps))
            C.gemm_i8_ex(h8, self.fc2.weight, res2d, self.fc2.bias, epilogue=C.EPI_F32_BIAS_F32_ACC,
                         m=res2d.shape[0], n=e, k=self.local_ffn, lda=self.local_ffn, ldb=self.local_ffn, ldc=e,
                         alpha=self.fc2._scalar("a"), beta=1.0)
            del h8
            if next_ln is None:
                return residual, None
            return residual, C.layernorm_q(residual, next_ln.weight, next_ln.bias, next_ln.eps)
        acc = attn.forward_fused(hidden_int8, cache, layer_idx, past_len, mask, decode=decode)
        acc = self.tp.all_reduce_int32(acc)
        ln = self.final_layer_norm
        residual, h8 = C.dq_add_layernorm_q_bias(acc.view(shape), attn.out_proj._scalar("a"), attn.out_proj.bias,
                                                 residual, ln.weight, ln.bias, ln.eps)
        del acc
        h8 = self.fc1._op(h8.view(-1, self.embed_dim))
        acc = torch.empty((h8.shape[0], self.embed_dim), dtype=torch.int32, device=h8.device)
        C.gemm_i8_ex(h8, self.fc2.weight, acc, epilogue=C.EPI_S32_RAW, m=h8.shape[0], n=self.embed_dim,
                     k=self.local_ffn, lda=self.local_ffn, ldb=self.local_ffn, ldc=self.embed_dim)
        del h8
        acc = self.tp.all_reduce_int32(acc)
        ln = next_ln if next_ln is not None else self._identity_ln(residual.device)
        residual, h8 = C.dq_add_layernorm_q_bias(acc.view(shape), self.fc2._scalar("a"), self.fc2.bias,
                                                 residual, ln.weight, ln.bias, ln.eps)
        return residual, (h8 if next_ln is not None else None)

    def _identity_ln(self, device):
        ln = getattr(self, "_id_ln", None)
        if ln is None or ln.weight.device != device:
            ln = LayerNormQ(self.embed_dim).to(device)
            object.__setattr__(self, "_id_ln", ln)
        return ln

    # ------------------------------------------------------- reference signature
    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                layer_head_mask: Optional[torch.Tensor] = None, output_attentions: Optional[bool] = False,
                use_cache: Optional[bool] = False, past_key_value: Optional[Tuple[torch.Tensor]] = None):
        """hidden_states: floating-point residual stream [B,T,E]; it is updated IN
        PLACE and returned, as in the reference (opt.py:270-289)."""
        residual = hidden_states
        hidden_states = self.self_attn_layer_norm(hidden_states)
        hidden_states, self_attn_weights, present_key_value = self.self_attn(
            hidden_states=hidden_states, past_key_value=past_key_value, attention_mask=attention_mask,
            layer_head_mask=layer_head_mask, output_attentions=output_attentions)
        residual.add_(hidden_states.to(residual.dtype))
        hidden_states = self.final_layer_norm(residual)
        hidden_states = self.fc1(hidden_states)
        hidden_states = self.fc2(hidden_states)
        residual.add_(hidden_states.to(residual.dtype))
        outputs = (residual,)
        if output_attentions:
            outputs += (self_attn_weights,)
        if use_cache:
            outputs += (present_key_value,)
        return outputs


class OPTLearnedPositions(nn.Embedding):
    """OPT's learned positions: ids are offset by 2 (a fairseq leftover that the
    checkpoints depend on); positions count only non-padding tokens."""

    def __init__(self, num_embeddings: int, embedding_dim: int):
        self.offset = 2
        super().__init__(num_embeddings + self.offset, embedding_dim)

    def forward(self, attention_mask: torch.LongTensor, past_key_values_length: int = 0):
        attention_mask = attention_mask.long()
        positions = (torch.cumsum(attention_mask, dim=1) * attention_mask).long() - 1
        positions = positions[:, past_key_values_length:]
        return super().forward(positions + self.offset)


@dataclass
class DecoderOutput:
    last_hidden_state: torch.Tensor
    past_key_values: Optional[StaticInt8KVCache] = None


@dataclass
class CausalLMOutput:
    logits: torch.Tensor
    past_key_values: Optional[StaticInt8KVCache] = None


class Int8OPTDecoder(nn.Module):
    """Embeddings + *config.num_hidden_layers* Int8OPTDecoderLayer + final LayerNorm
    (opt.py:302-398)."""

    def __init__(self, config, tp: Optional[TensorParallel] = None):
        super().__init__()
        self.config = config
        self.tp = tp if tp is not None else TensorParallel.single()
        self.padding_idx = config.pad_token_id
        self.max_target_positions = config.max_position_embeddings
        self.vocab_size = config.vocab_size
        proj = config.word_embed_proj_dim
        self.embed_tokens = nn.Embedding(config.vocab_size, proj, self.padding_idx)
        self.embed_positions = OPTLearnedPositions(config.max_position_embeddings, config.hidden_size)
        self.project_out = nn.Linear(config.hidden_size, proj, bias=False) if proj != config.hidden_size else None
        self.project_in = nn.Linear(proj, config.hidden_size, bias=False) if proj != config.hidden_size else None
        if config.do_layer_norm_before and not getattr(config, "_remove_final_layer_norm", False):
            self.final_layer_norm = nn.LayerNorm(config.hidden_size)
        else:
            self.final_layer_norm = None
        self.layers = nn.ModuleList([
            Int8OPTDecoderLayer(config.hidden_size, config.num_attention_heads, config.ffn_dim, tp=self.tp)
            for _ in range(config.num_hidden_layers)])
        # dtype of the residual stream between the layers.  torch.float32 (default): the embeddings are
        # widened once and every residual update is exact fp32 arithmetic.  None: the dtype of the
        # embeddings, as in the reference (opt.py:270-289 updates `hidden_states` in place), so a model
        # held in fp16 - the reference benchmark's default precision "int8-fp16" - keeps an fp16 residual
        # stream: each linear's fp32 output is cast to fp16 and added in fp16.  torch.float16 forces that.
        # Tensor-parallel runs always use fp32 (the exchange kernels reduce into fp32 rows).
        self.residual_dtype = torch.float32

    def get_input_embeddings(self):
        return self.embed_tokens

    def set_input_embeddings(self, value):
        self.embed_tokens = value

    @staticmethod
    def from_float(module, decoder_layer_scales):
        """Quantises a float OPTDecoder; `decoder_layer_scales[i]` holds the keyword
        arguments of Int8OPTDecoderLayer.from_float for layer i (opt.py:352-361)."""
        int8_module = Int8OPTDecoder(module.config)
        int8_module.embed_tokens = module.embed_tokens
        int8_module.embed_positions.weight = module.embed_positions.weight
        int8_module.project_out = module.project_out
        int8_module.project_in = module.project_in
        int8_module.final_layer_norm = module.final_layer_norm
        for i, layer in enumerate(module.layers):
            int8_module.layers[i] = Int8OPTDecoderLayer.from_float(layer, **decoder_layer_scales[i])
        return int8_module

    def new_cache(self, batch_size: int, max_len: int, device=None) -> StaticInt8KVCache:
        """Pre-allocated int8 key / transposed-value cache for `max_len` positions."""
        attn = self.layers[0].self_attn
        device = device if device is not None else self.embed_tokens.weight.device
        return StaticInt8KVCache(len(self.layers), batch_size, attn.local_heads, attn.head_dim, max_len, device)

    def _stream_dtype(self, hidden):
        """dtype of the residual stream for embeddings `hidden` (see residual_dtype)."""
        want = self.residual_dtype if self.residual_dtype is not None else hidden.dtype
        if self.tp.size > 1 or want not in (torch.float32, torch.float16):
            return torch.float32
        return want

    @staticmethod
    def _additive_mask(attention_mask, tgt_len, past_len, src_pad, dtype=torch.float32):
        """[B,1,T,src_pad] additive mask: causal + padding, finfo.min where hidden
        (what transformers' OPT decoder builds for the reference, opt.py:348)."""
        bsz, src_len = attention_mask.shape
        neg = torch.finfo(dtype).min
        dev = attention_mask.device
        rows = torch.arange(tgt_len, device=dev).view(tgt_len, 1) + past_len
        cols = torch.arange(src_pad, device=dev).view(1, src_pad)
        visible = (cols <= rows).view(1, 1, tgt_len, src_pad)
        keep = torch.zeros((bsz, src_pad), dtype=torch.bool, device=dev)
        keep[:, :src_len] = attention_mask.bool()
        visible = visible & keep.view(bsz, 1, 1, src_pad)
        mask = torch.full((bsz, 1, tgt_len, src_pad), neg, dtype=dtype, device=dev)
        return mask.masked_fill(visible, 0.0).contiguous()

    def _layers_pipelined(self, residual, cache, past_len, mask, chunks):
        """Tensor-parallel layer loop.  The batch is cut into `chunks` groups of whole
        sequences; per group and per exchange point the int32 partial sums are
        reduce-scattered over the ranks by token rows, the fused dequant + bias +
        residual add + LayerNorm-quantise runs on this rank's rows only (the residual
        stream stays sharded by tokens), and the int8 result is all-gathered: 5 bytes
        per element cross NVLink instead of the 8 of an all-reduce.  Communication runs
        on its own stream, so the exchange of one group overlaps the GEMMs of the next."""
        tp = self.tp
        n, rank = tp.size, tp.rank
        bsz, tgt_len, e = residual.shape
        bc = bsz // chunks
        mc = bc * tgt_len
        ms = mc // n
        dev = residual.device
        compute = torch.cuda.current_stream(dev)
        comm = tp.comm_stream(dev)
        layers = self.layers
        first = layers[0].self_attn_layer_norm
        ws = tp.peer_workspace(chunks, mc, e, dev)
        res, h8, acc, ready, done = [], [], [], [], []
        for c in range(chunks):
            full = residual[c * bc:(c + 1) * bc]
            q0 = C.layernorm_q(full, first.weight, first.bias, first.eps)
            if ws is not None:
                ws.h8[c].copy_(q0.view(mc, e))
                h8.append(ws.h8[c].view(bc, tgt_len, e))
                acc.append(torch.empty((mc, e), dtype=torch.int32, device=dev) if tp.peer_mode == "copy" else None)
            else:
                h8.append(q0)
                acc.append(torch.empty((mc, e), dtype=torch.int32, device=dev))
            res.append(full.reshape(mc, e)[rank * ms:(rank + 1) * ms].clone())
            res[c].record_stream(comm)  # first consumed (and released) on the communication stream
            ready.append(torch.cuda.Event())
            done.append(torch.cuda.Event())
            ready[c].record(compute)
        comm.wait_stream(compute)

        # with a second communication stream the reduction of one group overlaps the copies of the next
        comm2 = tp.comm_stream(dev, 1) if (ws is not None and tp.comm_streams > 1) else comm
        copied = [torch.cuda.Event() for _ in range(chunks)] if comm2 is not comm else None
        if comm2 is not comm:
            comm2.wait_stream(compute)
            for c in range(chunks):
                res[c].record_stream(comm2)

        def exchange(c, scale, bias, ln, tag):
            """On the communication stream(s).  Peer-memory form: this rank's partial sums go into
            the owners' stage slabs (copy engines, or already stored there by the GEMM epilogue), then
            ONE kernel announces them, waits for all ranks', sums the slabs of my rows, applies scale/
            bias/residual/LayerNorm/quantise, stores the int8 rows into every rank's activation buffer
            and ends when every rank has done so (tp.fused_sync; otherwise the same steps as barrier ->
            reduce kernel -> barrier).  NCCL form: reduce-scatter -> fused LayerNorm kernel -> all-gather."""
            done[c].record(compute)
            with torch.cuda.stream(comm):
                comm.wait_event(done[c])
                if ws is not None:
                    with tp.span("push", "exchange.copy", comm, group=c, at=tag):
                        if tp.peer_mode == "copy":
                            ws.push_partials(c, acc[c])
                        if not tp.fused_sync:
                            ws.barrier(0)
                    if comm2 is not comm:
                        copied[c].record(comm)
                else:
                    with tp.span("nccl", "exchange.copy", comm, group=c, at=tag):
                        shard = tp.reduce_scatter_int32(acc[c])
                        res[c], q = C.dq_add_layernorm_q_bias(shard, scale, bias, res[c], ln.weight, ln.bias, ln.eps)
                        tp.all_gather_into(h8[c].view(mc, e), q)
                    ready[c].record(comm)
            if ws is not None:
                with torch.cuda.stream(comm2):
                    if comm2 is not comm:
                        comm2.wait_event(copied[c])
                    if tp.fused_sync:
                        with tp.span("sync+reduce+ln+sync", "exchange.reduce", comm2, group=c, at=tag):
                            res[c] = ws.exchange_reduce(c, scale, bias, res[c], ln)
                    else:
                        with tp.span("reduce+ln", "exchange.reduce", comm2, group=c, at=tag):
                            res[c] = C.tp_reduce_layernorm_q(ws.stage[c], n, ms * e, scale, bias, res[c], ln.weight,
                                                             ln.bias, ln.eps, ws.q_dst_ptrs(c), rank * ms)
                        with tp.span("barrier", "exchange.reduce", comm2, group=c, at=tag):
                            ws.barrier(1 if comm2 is not comm else 0)
                    ready[c].record(comm2)

        def row_parallel(c, x2d, weight, k):
            """int32 partial sums of a row-parallel linear for chunk c: to the owners' stage slabs
            (peer stores from the GEMM epilogue) or to the local buffer for NCCL."""
            if ws is not None and tp.peer_mode != "copy":
                C.gemm_i8_ex(x2d, weight, None, epilogue=C.EPI_S32_RAW, m=mc, n=e, k=k, lda=k, ldb=k, ldc=e,
                             scatter_ptrs=ws.scatter_ptrs(c), scatter_rows=ms)
            else:
                C.gemm_i8_ex(x2d, weight, acc[c], epilogue=C.EPI_S32_RAW, m=mc, n=e, k=k, lda=k, ldb=k, ldc=e)

        nl = len(layers)
        for i, layer in enumerate(layers):
            attn = layer.self_attn
            for c in range(chunks):
                compute.wait_event(ready[c])
                with tp.span("attention+out_proj", "compute", compute, group=c, layer=i):
                    m = None if mask is None else mask[c * bc:(c + 1) * bc]
                    ctx = attn.forward_fused(h8[c], cache, i, past_len, m, b0=c * bc, context_only=True)
                    row_parallel(c, ctx.view(mc, attn.local_dim), attn.out_proj.weight, attn.local_dim)
                exchange(c, attn.out_proj._scalar("a"), attn.out_proj.bias, layer.final_layer_norm, f"{i}.attn")
            next_ln = layers[i + 1].self_attn_layer_norm if i + 1 < nl else layer._identity_ln(dev)
            for c in range(chunks):
                compute.wait_event(ready[c])
                with tp.span("fc1+fc2", "compute", compute, group=c, layer=i):
                    f8 = layer.fc1._op(h8[c].view(mc, e))
                    row_parallel(c, f8, layer.fc2.weight, layer.local_ffn)
                exchange(c, layer.fc2._scalar("a"), layer.fc2.bias, next_ln, f"{i}.ffn")
        out = torch.empty((bsz, tgt_len, e), dtype=torch.float32, device=dev)
        if comm2 is not comm:
            comm.wait_stream(comm2)
        with torch.cuda.stream(comm):
            for c in range(chunks):
                if comm2 is not comm:
                    res[c].record_stream(comm)  # allocated on the second stream, last read on this one
                tp.all_gather_into(out[c * bc:(c + 1) * bc].view(mc, e), res[c])
        compute.wait_stream(comm)
        if ws is not None and (not ws.checked or _CHECK_EVERY_PASS):
            # a barrier whose bounded wait ran out leaves the activations unsynchronised: find out now
            # (all ranks together) instead of returning wrong logits silently
            tp.check_exchange(ws, dev)
        return out

    @torch.no_grad()
    def decode_step(self, tokens: torch.LongTensor, cache: StaticInt8KVCache) -> torch.Tensor:
        """One new token per sequence ([B,1]) on top of `cache` (no padding tokens in the batch).
        Everything position dependent reads cache.pos on the device, so the whole step is a fixed
        sequence of launches with fixed arguments: it can be captured once in a CUDA graph and
        replayed.  Returns the last hidden state [B,1,proj]."""
        bsz = tokens.shape[0]
        if self.layers[0].self_attn.head_dim not in (64, 128):
            # the one-token attention kernel covers head_dim 64 and 128 (all OPT sizes but 2.7B, whose
            # heads are 80 wide); other widths take the prefill path with one query row per sequence,
            # which reads the position on the host and therefore cannot be replayed from a CUDA graph
            return self.forward(tokens, past_key_values=cache, use_cache=True).last_hidden_state
        hidden = self.embed_tokens(tokens)
        if self.project_in is not None:
            hidden = self.project_in(hidden)
        pos_ids = (cache.pos.long() + self.embed_positions.offset).view(1, 1).expand(bsz, 1)
        hidden = hidden + nn.functional.embedding(pos_ids, self.embed_positions.weight)
        residual = hidden.to(self._stream_dtype(hidden)).contiguous()
        first = self.layers[0].self_attn_layer_norm
        h8 = C.layernorm_q(residual, first.weight, first.bias, first.eps)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            next_ln = self.layers[i + 1].self_attn_layer_norm if i + 1 < n else None
            residual, h8 = layer.forward_fused(residual, h8, cache, i, None, None, next_ln, decode=True)
        C.advance_position(cache.pos, 1)
        cache.length += 1
        residual = residual.to(hidden.dtype)
        if self.final_layer_norm is not None:
            residual = self.final_layer_norm(residual)
        if self.project_out is not None:
            residual = self.project_out(residual)
        return residual

    @torch.no_grad()
    def forward(self, input_ids: torch.LongTensor, attention_mask: Optional[torch.Tensor] = None,
                past_key_values: Optional[StaticInt8KVCache] = None, use_cache: bool = False,
                reference_path: bool = False) -> DecoderOutput:
        """input_ids [B,T] -> last hidden state [B,T,proj].  The reference pads T to a
        multiple of 16 with <pad> tokens and slices the result (opt.py:375-397); here the
        key length is padded inside the attention instead, which leaves every real
        position's result unchanged.  `reference_path=True` runs the layers through their
        reference-signature forwards (single GPU, no cache, T a multiple of 16)."""
        bsz, tgt_len = input_ids.shape
        cache = past_key_values
        if use_cache and cache is None:
            cache = self.new_cache(bsz, self.max_target_positions, input_ids.device)
        past_len = cache.length if cache is not None else 0
        src_len = past_len + tgt_len
        if attention_mask is None:
            attention_mask_full = torch.ones((bsz, src_len), dtype=torch.long, device=input_ids.device)
            padding_free = True
        else:
            attention_mask_full = attention_mask
            padding_free = bool(attention_mask.bool().all())
        hidden = self.embed_tokens(input_ids)
        if self.project_in is not None:
            hidden = self.project_in(hidden)
        hidden = hidden + self.embed_positions(attention_mask_full, past_len)
        if not padding_free and src_len > attention_mask_full.shape[1]:
            raise ValueError("attention_mask must cover the cached and the new positions")
        src_pad = _round_up(src_len, 16)
        mask = None if padding_free else self._additive_mask(attention_mask_full, tgt_len, past_len, src_pad)

        if reference_path:
            if cache is not None or self.tp.size != 1:
                raise RuntimeError("reference_path supports neither a cache nor tensor parallelism")
            ref_mask = self._additive_mask(attention_mask_full, tgt_len, 0, src_len)
            residual = hidden.contiguous().clone()
            for layer in self.layers:
                residual = layer(residual, attention_mask=ref_mask)[0]
        else:
            residual = hidden.to(self._stream_dtype(hidden)).contiguous()
            owned = True  # `hidden` is this call's own sum of embeddings: the layers may update it in place
            chunks = self.tp.plan_chunks(bsz, tgt_len) if self.tp.size > 1 else 0
            if chunks:
                residual = self._layers_pipelined(residual, cache, past_len, mask, chunks)
            else:
                first = self.layers[0].self_attn_layer_norm
                h8 = C.layernorm_q(residual, first.weight, first.bias, first.eps)
                n = len(self.layers)
                for i, layer in enumerate(self.layers):
                    next_ln = self.layers[i + 1].self_attn_layer_norm if i + 1 < n else None
                    residual, h8 = layer.forward_fused(residual, h8, cache, i, past_len, mask, next_ln,
                                                       inplace=owned)
            if cache is not None:
                cache.set_length(src_len)
            residual = residual.to(hidden.dtype)
        if self.final_layer_norm is not None:
            residual = self.final_layer_norm(residual)
        if self.project_out is not None:
            residual = self.project_out(residual)
        return DecoderOutput(residual, cache if use_cache else None)


class Int8OPTModel(nn.Module):
    """Thin shell around the decoder (opt.py:401-417)."""

    def __init__(self, config, tp: Optional[TensorParallel] = None):
        super().__init__()
        self.config = config
        self.decoder = Int8OPTDecoder(config, tp=tp)

    def get_input_embeddings(self):
        return self.decoder.embed_tokens

    def set_input_embeddings(self, value):
        self.decoder.embed_tokens = value

    def get_decoder(self):
        return self.decoder

    def forward(self, input_ids, attention_mask=None, past_key_values=None, use_cache=False, reference_path=False):
        return self.decoder(input_ids, attention_mask=attention_mask, past_key_values=past_key_values,
                            use_cache=use_cache, reference_path=reference_path)

    @staticmethod
    def from_float(module, decoder_layer_scales):
        int8_module = Int8OPTModel(module.config)
        int8_module.decoder = Int8OPTDecoder.from_float(module.decoder, decoder_layer_scales)
        return int8_module

    @classmethod
    def from_pretrained(cls, directory, device="cuda", torch_dtype=None, tp: Optional[TensorParallel] = None,
                        strict: bool = True, device_map=None):
        """Loads a checkpoint directory in the transformers layout (config.json + state-dict files with
        the reference's buffer names), as the reference's inherited ``from_pretrained`` does
        (benchmark/bench_opt.py:35-40).  With `tp`, each rank reads only its slices of the split weights."""
        from .checkpoint import load_pretrained
        return load_pretrained(cls, directory, device=device, torch_dtype=torch_dtype, tp=tp, strict=strict,
                               device_map=device_map)

    def save_pretrained(self, directory, max_shard_bytes: int = 5 << 30, safe_serialization: bool = True):
        from .checkpoint import save_pretrained
        return save_pretrained(self, directory, max_shard_bytes, safe_serialization)


class Int8OPTForCausalLM(nn.Module):
    """Int8 OPT with the language-model head, which is tied to the token embeddings
    and stays floating point (opt.py:420-450)."""

    _keys_to_ignore_on_load_missing = [r"lm_head.weight"]

    def __init__(self, config, tp: Optional[TensorParallel] = None):
        super().__init__()
        self.config = config
        self.model = Int8OPTModel(config, tp=tp)
        self.lm_head = nn.Linear(config.word_embed_proj_dim, config.vocab_size, bias=False)
        self.lm_head.weight = self.model.decoder.embed_tokens.weight  # tied

    @staticmethod
    def from_float(module, decoder_layer_scales):
        int8_module = Int8OPTForCausalLM(module.config)
        int8_module.model = Int8OPTModel.from_float(module.model, decoder_layer_scales)
        int8_module.lm_head = module.lm_head
        return int8_module

    @classmethod
    def from_pretrained(cls, directory, device="cuda", torch_dtype=None, tp: Optional[TensorParallel] = None,
                        strict: bool = True, device_map=None):
        """Loads a checkpoint directory in the transformers layout (config.json + state-dict files with
        the reference's buffer names), as the reference's inherited ``from_pretrained`` does
        (benchmark/bench_opt.py:35-40).  With `tp`, each rank reads only its slices of the split weights."""
        from .checkpoint import load_pretrained
        return load_pretrained(cls, directory, device=device, torch_dtype=torch_dtype, tp=tp, strict=strict,
                               device_map=device_map)

    def save_pretrained(self, directory, max_shard_bytes: int = 5 << 30, safe_serialization: bool = True):
        from .checkpoint import save_pretrained
        return save_pretrained(self, directory, max_shard_bytes, safe_serialization)

    def get_input_embeddings(self):
        return self.model.decoder.embed_tokens

    def set_input_embeddings(self, value):
        self.model.decoder.embed_tokens = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new_embeddings):
        self.lm_head = new_embeddings

    def set_decoder(self, decoder):
        self.model.decoder = decoder

    def get_decoder(self):
        return self.model.decoder

    def new_cache(self, batch_size, max_len, device=None):
        return self.model.decoder.new_cache(batch_size, max_len, device)

    @torch.no_grad()
    def forward(self, input_ids, attention_mask=None, past_key_values=None, use_cache=False,
                reference_path=False, last_token_only=False) -> CausalLMOutput:
        out = self.model(input_ids, attention_mask=attention_mask, past_key_values=past_key_values,
                         use_cache=use_cache, reference_path=reference_path)
        hidden = out.last_hidden_state
        if last_token_only:
            hidden = hidden[:, -1:, :]
        return CausalLMOutput(self._logits(hidden).contiguous(), out.past_key_values)

    def _logits(self, hidden):
        hidden = hidden.to(self.lm_head.weight.dtype)
        tp = self.model.decoder.tp
        if tp.size > 1 and tp.vocab_parallel and self.lm_head.bias is None:
            return tp.vocab_parallel_logits(hidden, self.lm_head.weight)
        return self.lm_head(hidden)

    @torch.no_grad()
    def decode_step(self, tokens, cache: StaticInt8KVCache):
        """Logits [B, vocab] of the token after `tokens` [B,1], appended to `cache`."""
        hidden = self.model.decoder.decode_step(tokens, cache)
        return self._logits(hidden[:, -1, :])

    @torch.no_grad()
    def generate_greedy(self, input_ids, max_new_tokens: int, cache: Optional[StaticInt8KVCache] = None,
                        use_cuda_graph: Optional[bool] = None):
        """Prefill + greedy decoding with the static int8 cache.  Returns [B, T + new].
        With use_cuda_graph (default on a single GPU) the decode step is captured once per cache -
        after a first eager step has initialised everything lazy - and replayed for the other steps."""
        bsz, t = input_ids.shape
        if cache is None:
            cache = self.new_cache(bsz, t + max_new_tokens)
        else:
            cache.reset()
        if t + max_new_tokens > cache.capacity:
            raise RuntimeError(f"cache capacity {cache.capacity} is too small for {t} + {max_new_tokens} tokens")
        dec = self.model.decoder
        # tensor-parallel steps contain NCCL all-reduces; capturing them needs every rank to capture and
        # replay in lockstep, which generate_greedy does (opt-in: TensorParallel.decode_graph)
        graph_ok = (dec.tp.size == 1 or dec.tp.decode_graph) and dec.layers[0].self_attn.head_dim in (64, 128)
        if use_cuda_graph is None:
            use_cuda_graph = graph_ok
        use_cuda_graph = use_cuda_graph and graph_ok
        out = self.forward(input_ids, past_key_values=cache, use_cache=True, last_token_only=True)
        tokens = [input_ids]
        nxt = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)
        steps_left = max_new_tokens - 1
        if steps_left > 0:  # first decode step eagerly (also warms up everything a capture must not do)
            tokens.append(nxt)
            nxt = self.decode_step(nxt, cache).argmax(dim=-1, keepdim=True)
            steps_left -= 1
        if use_cuda_graph and steps_left > 0:
            if cache.graph is None or cache.graph[1].shape != nxt.shape:
                static_tok = nxt.clone()
                length = cache.length
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    static_next = self.decode_step(static_tok, cache).argmax(dim=-1, keepdim=True)
                cache.length = length  # capturing records the step, it does not run it
                cache.graph = (graph, static_tok, static_next)
            graph, static_tok, static_next = cache.graph
            for _ in range(steps_left):
                tokens.append(nxt)
                static_tok.copy_(nxt)
                graph.replay()
                cache.length += 1
                nxt = static_next.clone()
        else:
            for _ in range(steps_left):
                tokens.append(nxt)
                nxt = self.decode_step(nxt, cache).argmax(dim=-1, keepdim=True)
        tokens.append(nxt)
        return torch.cat(tokens, dim=1)
