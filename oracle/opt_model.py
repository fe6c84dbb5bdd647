"""TEST INFRASTRUCTURE: CPU restatement of the reference's Int8 OPT dataflow.

Follows torch_int/models/opt.py step by step - Int8OPTAttention.forward
(opt.py:83-199), Int8OPTDecoderLayer.forward (opt.py:244-299) and the decoder
shell (opt.py:363-398, whose embedding / position / mask / final-LayerNorm
logic the reference borrows from transformers' OPTDecoder) - with every op
evaluated by the CPU oracle (oracle/w8a8.py).  Parameters come from a state
dict with the reference's names, e.g.
``model.decoder.layers.0.self_attn.q_proj.weight``.

Model-level parity is unpinned by the reference itself: its model tests print
an error metric without a threshold and need checkpoints that are not
available offline; this emulation of its code path is the pin.

Never imported by the product.
"""
import torch

from . import w8a8 as O


def _f(sd, name):
    return float(sd[name])


def _linear_s8(sd, prefix, x2d, relu=False):
    fn = O.linear_relu_a8_w8_b8_o8 if relu else O.linear_a8_w8_b8_o8
    return fn(x2d, sd[prefix + ".weight"], sd[prefix + ".bias"], _f(sd, prefix + ".a"), _f(sd, prefix + ".b"))


def _linear_f32(sd, prefix, x2d):
    # W8A8BFP32OFP32Linear.forward passes beta = 1 (torch_int/nn/linear.py:213-214)
    return O.linear_a8_w8_bfp32_ofp32(x2d, sd[prefix + ".weight"], sd[prefix + ".bias"].float(),
                                      _f(sd, prefix + ".a"), 1.0)


def attention(sd, prefix, hidden_int8, mask, num_heads, past=None, trace=None):
    """Int8OPTAttention.forward (opt.py:83-199).  hidden_int8 [B,T,E] int8, mask
    additive [B,1,T,S] or None, past = (k, v) int8 [B,H,S0,D] or None.
    Returns (fp32 [B,T,E], (k, v)).  `trace`: optional dict that receives the int8 tensors between the
    ops (q, k, v [B*H,*,D], probs [B*H,T,S], ctx [B,T,E])."""
    bsz, tgt, e = hidden_int8.shape
    d = e // num_heads
    x2d = hidden_int8.reshape(-1, e)

    def shape(t):  # opt.py:80-81
        return t.view(bsz, -1, num_heads, d).transpose(1, 2).contiguous()

    q = shape(_linear_s8(sd, prefix + ".q_proj", x2d))
    k = shape(_linear_s8(sd, prefix + ".k_proj", x2d))
    v = shape(_linear_s8(sd, prefix + ".v_proj", x2d))
    if past is not None:  # opt.py:113-116
        k = torch.cat([past[0], k], dim=2)
        v = torch.cat([past[1], v], dim=2)
    present = (k, v)
    q, k, v = (t.reshape(bsz * num_heads, -1, d) for t in (q, k, v))
    scores = O.bmm_s8t_s8n_f32t(q, k, _f(sd, prefix + ".qk_bmm.a"))              # opt.py:131
    probs = O.softmax_q(scores, mask)                                            # opt.py:139-178
    ctx = O.bmm_s8t_s8n_s8t(probs, v.transpose(1, 2).contiguous(), _f(sd, prefix + ".pv_bmm.a"))  # :180-181
    ctx = ctx.view(bsz, num_heads, tgt, d).transpose(1, 2).reshape(bsz, tgt, e).contiguous()      # :189-196
    out = _linear_f32(sd, prefix + ".out_proj", ctx.view(-1, e)).view(bsz, tgt, e)                 # :197
    if trace is not None:
        trace.update(q=q, k=k, v=v, probs=probs, ctx=ctx)
    return out, present


def decoder_layer(sd, prefix, hidden, mask, num_heads, past=None, eps=1e-5, trace=None):
    """Int8OPTDecoderLayer.forward (opt.py:270-289): returns (residual, present kv).  `trace`: optional
    dict that receives the tensors between the ops (ln1, q, k, v, probs, ctx, res1, ln2, fc1)."""
    residual = hidden.clone()
    h8 = O.layernorm_q(residual, sd[prefix + ".self_attn_layer_norm.weight"],
                       sd[prefix + ".self_attn_layer_norm.bias"], eps)
    if trace is not None:
        trace["ln1"] = h8
    attn_out, present = attention(sd, prefix + ".self_attn", h8, mask, num_heads, past, trace)
    residual.add_(attn_out.to(residual.dtype))
    h8 = O.layernorm_q(residual, sd[prefix + ".final_layer_norm.weight"], sd[prefix + ".final_layer_norm.bias"], eps)
    if trace is not None:
        trace.update(res1=residual.clone(), ln2=h8)
    bsz, tgt, e = h8.shape
    h8 = _linear_s8(sd, prefix + ".fc1", h8.view(-1, e), relu=True)
    if trace is not None:
        trace["fc1"] = h8
    h = _linear_f32(sd, prefix + ".fc2", h8).view(bsz, tgt, e)
    residual.add_(h.to(residual.dtype))
    return residual, present


def additive_mask(attention_mask, tgt_len, past_len, dtype=torch.float32):
    """Causal + padding mask [B,1,T,S] with finfo.min where hidden, as transformers'
    OPT decoder prepares it for the layers."""
    bsz, src = attention_mask.shape
    neg = torch.finfo(dtype).min
    rows = torch.arange(tgt_len).view(tgt_len, 1) + past_len
    cols = torch.arange(src).view(1, src)
    visible = (cols <= rows).view(1, 1, tgt_len, src) & attention_mask.bool().view(bsz, 1, 1, src)
    return torch.full((bsz, 1, tgt_len, src), neg, dtype=dtype).masked_fill(visible, 0.0)


def decoder(sd, config, input_ids, attention_mask=None, prefix="model.decoder", past=None):
    """Embeddings -> layers -> final LayerNorm.  No padding of the sequence to a
    multiple of 16 (opt.py:375-383 is an alignment work-around of the CUDA kernels;
    padded positions are masked out and sliced off again, so the result for the real
    positions is the same).  Returns (hidden [B,T,proj], list of present kv)."""
    bsz, tgt = input_ids.shape
    past_len = past[0][0].shape[2] if past is not None else 0
    src = past_len + tgt
    if attention_mask is None:
        attention_mask = torch.ones((bsz, src), dtype=torch.long)
    hidden = torch.nn.functional.embedding(input_ids, sd[prefix + ".embed_tokens.weight"])
    if prefix + ".project_in.weight" in sd:
        hidden = torch.nn.functional.linear(hidden, sd[prefix + ".project_in.weight"])
    am = attention_mask.long()
    positions = (torch.cumsum(am, dim=1) * am).long() - 1
    positions = positions[:, past_len:] + 2  # OPT's position offset
    hidden = hidden + torch.nn.functional.embedding(positions, sd[prefix + ".embed_positions.weight"])
    mask = additive_mask(attention_mask, tgt, past_len)
    residual = hidden.to(torch.float32)
    presents = []
    for i in range(config.num_hidden_layers):
        residual, present = decoder_layer(sd, f"{prefix}.layers.{i}", residual, mask, config.num_attention_heads,
                                          past[i] if past is not None else None)
        presents.append(present)
    residual = residual.to(hidden.dtype)
    if prefix + ".final_layer_norm.weight" in sd:
        residual = torch.nn.functional.layer_norm(residual, residual.shape[-1:], sd[prefix + ".final_layer_norm.weight"],
                                                  sd[prefix + ".final_layer_norm.bias"], 1e-5)
    if prefix + ".project_out.weight" in sd:
        residual = torch.nn.functional.linear(residual, sd[prefix + ".project_out.weight"])
    return residual, presents


def causal_lm_logits(sd, config, input_ids, attention_mask=None, past=None):
    hidden, presents = decoder(sd, config, input_ids, attention_mask, "model.decoder", past)
    w = sd["lm_head.weight"] if "lm_head.weight" in sd else sd["model.decoder.embed_tokens.weight"]
    return torch.nn.functional.linear(hidden.to(w.dtype), w), presents


# ----------------------------------------------------------- tensor-parallel restatement
def row_parallel_partial(x2d_shard, w_shard):
    """int32 partial sums of one rank of a row-parallel linear (the A4/A8 form)."""
    return O.gemm_acc(x2d_shard, w_shard)


def decoder_layer_tp(shards, prefix, hidden, mask, num_heads, eps=1e-5):
    """One decoder layer evaluated as `len(shards)` tensor-parallel ranks would:
    column-parallel q/k/v/fc1 on each rank's state-dict shard, int32 partial sums of
    out_proj/fc2 added over the ranks, then scale + bias + residual add once.  With
    fp32 activations this equals decoder_layer() on the unsharded state dict."""
    tp = len(shards)
    bsz, tgt, e = hidden.shape
    hl = num_heads // tp
    d = e // num_heads
    residual = hidden.clone()
    sd0 = shards[0]
    h8 = O.layernorm_q(residual, sd0[prefix + ".self_attn_layer_norm.weight"],
                       sd0[prefix + ".self_attn_layer_norm.bias"], eps)
    x2d = h8.view(-1, e)
    total = None
    for sd in shards:
        p = prefix + ".self_attn"

        def shape(t):
            return t.view(bsz, tgt, hl, d).transpose(1, 2).reshape(bsz * hl, tgt, d).contiguous()

        q, k, v = (shape(_linear_s8(sd, f"{p}.{n}", x2d)) for n in ("q_proj", "k_proj", "v_proj"))
        probs = O.softmax_q(O.bmm_s8t_s8n_f32t(q, k, _f(sd, p + ".qk_bmm.a")), mask)
        ctx = O.bmm_s8t_s8n_s8t(probs, v.transpose(1, 2).contiguous(), _f(sd, p + ".pv_bmm.a"))
        ctx = ctx.view(bsz, hl, tgt, d).transpose(1, 2).reshape(bsz * tgt, hl * d).contiguous()
        part = row_parallel_partial(ctx, sd[p + ".out_proj.weight"])
        total = part if total is None else total + part
    residual, h8 = O.dq_add_layernorm_q_bias(total.view(bsz, tgt, e), _f(sd0, prefix + ".self_attn.out_proj.a"),
                                             sd0[prefix + ".self_attn.out_proj.bias"].reshape(-1).float(), residual,
                                             sd0[prefix + ".final_layer_norm.weight"],
                                             sd0[prefix + ".final_layer_norm.bias"], eps)
    total = None
    for sd in shards:
        f8 = _linear_s8(sd, prefix + ".fc1", h8.view(-1, e), relu=True)
        part = row_parallel_partial(f8, sd[prefix + ".fc2.weight"])
        total = part if total is None else total + part
    ident_w, ident_b = torch.ones(e), torch.zeros(e)
    residual, _ = O.dq_add_layernorm_q_bias(total.view(bsz, tgt, e), _f(sd0, prefix + ".fc2.a"),
                                            sd0[prefix + ".fc2.bias"].reshape(-1).float(), residual, ident_w, ident_b, eps)
    return residual
