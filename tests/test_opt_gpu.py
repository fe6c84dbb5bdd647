"""Int8 OPT attention / decoder layer / causal LM on the GPU against the CPU
restatement of the reference's dataflow (oracle/opt_model.py)."""
import pytest
import torch

from helpers import assert_bit_exact, rand_s8, randn, set_fused_attention, set_residual_in_gemm
from oracle import opt_model as OM
from oracle import w8a8 as O

pytestmark = pytest.mark.gpu


def cpu_sd(model):
    sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    sd.setdefault("lm_head.weight", sd["model.decoder.embed_tokens.weight"])
    return sd


def small_model(layers=3, hidden=256, heads=4, ffn=1024, vocab=512, seed=0):
    from torch_int.models.opt import Int8OPTConfig
    from torch_int.models.random_init import random_int8_opt
    cfg = Int8OPTConfig(vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers, ffn_dim=ffn,
                        num_attention_heads=heads, max_position_embeddings=512)
    return cfg, random_int8_opt(cfg, seed=seed, device="cuda")


def rel_err(got, want):
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


@pytest.mark.parametrize("bsz,seq,dim,heads", [(1, 16, 16, 1), (2, 48, 256, 4), (1, 128, 512, 4)])
def test_attention_reference_signature(cuda_ops, bsz, seq, dim, heads):
    # B, L, D, H = 1, 16, 16, 1 is the shape of the reference's tests/test_opt_attention.py:21
    cfg, model = small_model(layers=1, hidden=dim, heads=heads, ffn=4 * dim)
    attn = model.model.decoder.layers[0].self_attn
    sd = cpu_sd(model)
    x = rand_s8((bsz, seq, dim), 1, -40, 40)
    mask = O.causal_mask(bsz, seq, seq)
    out, probs, (k, v) = attn(x.cuda(), attention_mask=mask.cuda())
    want, (k_o, v_o) = OM.attention(sd, "model.decoder.layers.0.self_attn", x, mask, heads)
    assert probs is None and out.dtype == torch.float32 and out.shape == (bsz, seq, dim)
    assert_bit_exact(k, k_o, "key states")
    assert_bit_exact(v, v_o, "value states")
    assert rel_err(out, want) < 2e-2  # probabilities may differ by one LSB at rounding ties
    # the optional outputs follow the reference's torch formulation
    out2, probs2, _ = attn(x.cuda(), attention_mask=mask.cuda(), output_attentions=True)
    assert probs2.shape == (bsz, heads, seq, seq) and rel_err(out2, want) < 2e-2
    assert torch.allclose(probs2.sum(-1), torch.ones_like(probs2.sum(-1)), atol=1e-5)


def test_attention_with_past_key_values(cuda_ops):
    cfg, model = small_model(layers=1, hidden=256, heads=4)
    attn = model.model.decoder.layers[0].self_attn
    sd = cpu_sd(model)
    x0, x1 = rand_s8((2, 32, 256), 2, -40, 40), rand_s8((2, 16, 256), 3, -40, 40)
    _, _, past = attn(x0.cuda(), attention_mask=O.causal_mask(2, 32, 32).cuda())
    mask = O.causal_mask(2, 16, 48)
    out, _, (k, v) = attn(x1.cuda(), past_key_value=past, attention_mask=mask.cuda())
    _, past_o = OM.attention(sd, "model.decoder.layers.0.self_attn", x0, O.causal_mask(2, 32, 32), 4)
    want, (k_o, _) = OM.attention(sd, "model.decoder.layers.0.self_attn", x1, mask, 4, past=past_o)
    assert k.shape == (2, 4, 48, 64)
    assert_bit_exact(k, k_o)
    assert rel_err(out, want) < 2e-2


def test_decoder_layer_both_wirings(cuda_ops):
    """Reference-signature forward (LayerNormQ -> attention -> residual.add_ -> ...) and the fused
    wiring (int32 GEMM output -> dq_add_layernorm_q) against the oracle, and against each other."""
    cfg, model = small_model(layers=2, hidden=512, heads=4, ffn=2048)
    set_fused_attention(model, False)  # both wirings on the same three attention kernels: bit-identical
    dec = model.model.decoder
    layer = dec.layers[0]
    sd = cpu_sd(model)
    bsz, seq = 2, 64
    hidden = randn((bsz, seq, 512), 5)
    mask = O.causal_mask(bsz, seq, seq)
    inp = hidden.cuda().clone()
    out_ref = layer(inp, attention_mask=mask.cuda())[0]
    assert out_ref.data_ptr() == inp.data_ptr(), "the residual is updated in place (opt.py:281,289)"
    want, _ = OM.decoder_layer(sd, "model.decoder.layers.0", hidden, mask, 4)
    assert rel_err(out_ref, want) < 1e-2
    ln = layer.self_attn_layer_norm
    h8 = cuda_ops.layernorm_q(hidden.cuda(), ln.weight, ln.bias, ln.eps)
    out_fused, h8_next = layer.forward_fused(hidden.cuda(), h8, None, 0, 0, None, dec.layers[1].self_attn_layer_norm)
    assert_bit_exact(out_fused.view(torch.int32), out_ref.view(torch.int32), "fused vs reference wiring")
    ln1 = dec.layers[1].self_attn_layer_norm
    assert_bit_exact(h8_next, cuda_ops.layernorm_q(out_fused, ln1.weight, ln1.bias, ln1.eps), "fused LN output")


def test_decoder_layer_opt13b_dims(cuda_ops):
    """hidden 5120, 40 heads, FFN 20480 (the OPT-13B layer), batch 1 x 512 tokens, against the oracle."""
    cfg, model = small_model(layers=1, hidden=5120, heads=40, ffn=20480, vocab=64)
    layer = model.model.decoder.layers[0]
    sd = cpu_sd(model)
    hidden = randn((1, 512, 5120), 6)
    mask = O.causal_mask(1, 512, 512)
    out = layer(hidden.cuda().clone(), attention_mask=mask.cuda())[0]
    want, _ = OM.decoder_layer(sd, "model.decoder.layers.0", hidden, mask, 40)
    assert rel_err(out, want) < 1e-2
    assert cuda_ops.device_status() == 0


def _stagewise_layer_check(C, model, hidden, heads, what):
    """Every op of one decoder layer, fed with the ORACLE's tensor of the previous stage, against the
    oracle's tensor of this stage: integer GEMM stages bit for bit, LayerNorm / softmax stages within one
    unit at rounding ties (>= 99.9 % identical), fp32 residuals bit for bit.  A wrong scale, bias or head
    offset anywhere in the layer's wiring fails its stage outright.  Then the layer as a whole."""
    from helpers import assert_quant_close
    layer = model.model.decoder.layers[0]
    attn = layer.self_attn
    sd = cpu_sd(model)
    bsz, seq, e = hidden.shape
    d = e // heads
    mask = O.causal_mask(bsz, seq, seq)
    tr = {}
    want, _ = OM.decoder_layer(sd, "model.decoder.layers.0", hidden, mask, heads, trace=tr)
    ln1, ln2 = layer.self_attn_layer_norm, layer.final_layer_norm
    assert_quant_close(C.layernorm_q(hidden.cuda(), ln1.weight, ln1.bias, ln1.eps), tr["ln1"], what=what + " ln1")
    x = tr["ln1"].cuda()

    def heads_first(t):                       # [B,T,E] -> [B*H,T,D]
        return t.view(bsz, seq, heads, d).transpose(1, 2).reshape(bsz * heads, seq, d).contiguous()
    for name, proj in (("q", attn.q_proj), ("k", attn.k_proj), ("v", attn.v_proj)):
        assert_bit_exact(heads_first(proj(x)), tr[name], f"{what} {name}_proj")
    q, k, v = tr["q"].cuda(), tr["k"].cuda(), tr["v"].cuda()
    probs = C.softmax_q(attn.qk_bmm(q, k), None, heads, causal=0)
    assert_quant_close(probs, tr["probs"], what=what + " probabilities")
    ctx3 = attn.pv_bmm(tr["probs"].cuda(), v.transpose(1, 2).contiguous())
    ctx3 = ctx3.view(bsz, heads, seq, d).transpose(1, 2).reshape(bsz, seq, e)
    assert_bit_exact(ctx3, tr["ctx"], what + " context (P.V)")
    # the one-kernel attention on the oracle's q, k, v: a probability that flips at a tie moves a context
    # value by at most alpha_pv * 127
    rows = lambda t: t.view(bsz, heads, seq, d).transpose(1, 2).reshape(bsz, seq, e).contiguous()  # noqa: E731
    out = torch.empty((bsz, seq, e), dtype=torch.int8, device="cuda")
    C.attention_prefill(rows(q), rows(k), v.view(bsz, heads, seq, d).transpose(2, 3).contiguous(), out, batch=bsz,
                        heads=heads, head_dim=d, tgt_len=seq, src_len=seq, ld_q=e, q_batch_stride=seq * e, ld_k=e,
                        k_batch_stride=seq * e, ld_vt=seq, alpha_qk=attn.qk_bmm._alpha(), alpha_pv=attn.pv_bmm._alpha())
    dctx = (out.cpu().int() - tr["ctx"].int()).abs()
    assert float((dctx == 0).double().mean()) >= 0.995, what + " fused attention context"
    assert int(dctx.max()) <= int(abs(attn.pv_bmm._alpha()) * 127) + 1
    # out_proj as int32 partial sums + scale + bias + residual add + LayerNorm-quantise
    acc = torch.empty((bsz * seq, e), dtype=torch.int32, device="cuda")
    C.gemm_i8_ex(tr["ctx"].cuda().view(-1, e), attn.out_proj.weight, acc, epilogue=C.EPI_S32_RAW, m=bsz * seq, n=e,
                 k=e, lda=e, ldb=e, ldc=e)
    res1, h8 = C.dq_add_layernorm_q_bias(acc.view(bsz, seq, e), attn.out_proj._scalar("a"), attn.out_proj.bias,
                                         hidden.cuda(), ln2.weight, ln2.bias, ln2.eps)
    assert_bit_exact(res1.view(torch.int32), tr["res1"].view(torch.int32), what + " residual after attention")
    assert_quant_close(h8, tr["ln2"], what=what + " ln2")
    f8 = layer.fc1(tr["ln2"].cuda().view(-1, e))
    assert_bit_exact(f8, tr["fc1"], what + " fc1")
    C.gemm_i8_ex(f8, layer.fc2.weight, acc, epilogue=C.EPI_S32_RAW, m=bsz * seq, n=e, k=f8.shape[1],
                 lda=f8.shape[1], ldb=f8.shape[1], ldc=e)
    ident = layer._identity_ln(torch.device("cuda"))
    res2, _ = C.dq_add_layernorm_q_bias(acc.view(bsz, seq, e), layer.fc2._scalar("a"), layer.fc2.bias,
                                        tr["res1"].cuda(), ident.weight, ident.bias, ident.eps)
    # fed with the oracle's fc1 output and residual, the layer's output is the oracle's bit for bit
    assert_bit_exact(res2.view(torch.int32), want.view(torch.int32), what + " layer output (stage-wise)")
    # ... and the layer as a whole (tie flips of earlier stages propagate: a relative bound)
    whole = layer(hidden.cuda().clone(), attention_mask=mask.cuda())[0]
    assert rel_err(whole, want) < 1e-2
    assert C.device_status() == 0


def test_layer_stagewise_opt13b_batch4(cuda_ops):
    """Int8OPTDecoderLayer at the OPT-13B dimensions (hidden 5120, 40 heads, FFN 20480), batch 4 x 512."""
    cfg, model = small_model(layers=1, hidden=5120, heads=40, ffn=20480, vocab=64)
    _stagewise_layer_check(cuda_ops, model, randn((4, 512, 5120), 16), 40, "OPT-13B layer")


def test_layer_stagewise_opt30b(cuda_ops):
    """One layer at the OPT-30B dimensions (hidden 7168, 56 heads, FFN 28672), 1 x 512 tokens."""
    cfg, model = small_model(layers=1, hidden=7168, heads=56, ffn=28672, vocab=64)
    _stagewise_layer_check(cuda_ops, model, randn((1, 512, 7168), 17), 56, "OPT-30B layer")


def test_layer_stagewise_small(cuda_ops):
    cfg, model = small_model(layers=1, hidden=512, heads=4, ffn=2048)
    _stagewise_layer_check(cuda_ops, model, randn((2, 192, 512), 18), 4, "small layer")


@pytest.mark.parametrize("seq", [64, 255])
def test_causal_lm_logits(cuda_ops, seq):
    # L = 255 exercises a sequence length that is not a multiple of 16, as the
    # reference's tests/test_opt_decoder.py:30 does for its padding path.
    cfg, model = small_model()
    sd = cpu_sd(model)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, cfg.vocab_size, (2, seq), generator=g)
    logits = model(ids.cuda()).logits
    want, _ = OM.causal_lm_logits(sd, cfg, ids)
    assert logits.shape == (2, seq, cfg.vocab_size)
    assert rel_err(logits, want) < 2e-2
    assert float((logits.argmax(-1).cpu() == want.argmax(-1)).double().mean()) > 0.97
    if seq % 16 == 0:
        # with the same three attention kernels on both sides the two wirings agree bit for bit
        set_fused_attention(model, False)
        ref_path = model(ids.cuda(), reference_path=True).logits
        unfused = model(ids.cuda()).logits
        assert_bit_exact(ref_path.view(torch.int32), unfused.view(torch.int32), "reference-signature layers vs fused wiring")
        assert rel_err(unfused, logits) < 1e-2   # one-kernel attention: tie flips only


def test_residual_added_in_the_gemm_epilogue(cuda_ops):
    """Prefill with more than 128 tokens on one GPU adds the out_proj / fc2 outputs to the fp32 residual in the
    GEMM epilogue.  Bit for bit the same logits as with the fused residual/LayerNorm row kernel, and as the
    reference-signature layers."""
    cfg, model = small_model()
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, cfg.vocab_size, (3, 96), generator=g).cuda()
    set_fused_attention(model, False)
    in_gemm = model(ids).logits
    set_residual_in_gemm(model, False)
    in_row_kernel = model(ids).logits
    ref_path = model(ids, reference_path=True).logits
    assert_bit_exact(in_gemm.view(torch.int32), in_row_kernel.view(torch.int32), "residual add in the GEMM epilogue")
    assert_bit_exact(in_gemm.view(torch.int32), ref_path.view(torch.int32), "reference-signature layers")
    set_fused_attention(model, True)
    a = model(ids).logits
    set_residual_in_gemm(model, True)
    b = model(ids).logits
    assert_bit_exact(a.view(torch.int32), b.view(torch.int32), "with the one-kernel attention")
    cache = model.new_cache(3, 128)   # with a cache: prefill through the new path, then one decode step
    out = model(ids, past_key_values=cache, use_cache=True, last_token_only=True)
    set_residual_in_gemm(model, False)
    cache2 = model.new_cache(3, 128)
    out2 = model(ids, past_key_values=cache2, use_cache=True, last_token_only=True)
    assert_bit_exact(out.logits.view(torch.int32), out2.logits.view(torch.int32), "prefill into a cache")
    assert cuda_ops.device_status() == 0


def test_fp16_residual_stream(cuda_ops):
    """A model held in fp16 (the reference benchmark's default precision, int8-fp16): with residual_dtype =
    None the fused wiring keeps the residual stream in fp16 exactly as the reference-signature layers do
    (bit-identical logits with the same attention kernels), and agrees with the oracle's fp16 evaluation."""
    from torch_int.models.opt import Int8OPTConfig
    from torch_int.models.random_init import random_int8_opt
    cfg = Int8OPTConfig(vocab_size=512, hidden_size=256, num_hidden_layers=3, ffn_dim=1024, num_attention_heads=4,
                        max_position_embeddings=512)
    model = random_int8_opt(cfg, seed=4, device="cuda", param_dtype=torch.float16)
    sd = cpu_sd(model)
    ids = torch.randint(0, cfg.vocab_size, (2, 64), generator=torch.Generator().manual_seed(3))
    dec = model.model.decoder
    assert dec.residual_dtype == torch.float32
    fp32_stream = model(ids.cuda()).logits
    dec.residual_dtype = None                      # follow the embeddings, as the reference does
    set_fused_attention(model, False)
    got = model(ids.cuda()).logits
    ref_path = model(ids.cuda(), reference_path=True).logits
    assert got.dtype == torch.float16
    assert_bit_exact(got.view(torch.int16), ref_path.view(torch.int16), "fp16 residual: fused vs reference wiring")
    want, _ = OM.causal_lm_logits(sd, cfg, ids)    # fp16 embeddings -> the oracle's residual stream is fp16 too
    # (an fp16 stream rounds every residual update to 11 bits: looser than the fp32 comparisons)
    assert want.dtype == torch.float16 and rel_err(got, want) < 4e-2
    assert rel_err(got, fp32_stream) < 4e-2 and not torch.equal(got, fp32_stream)
    # decode steps on the fp16 stream reproduce the full forward
    set_fused_attention(model, True)
    out = model.generate_greedy(ids[:, :20].cuda(), 5)
    full = model(out[:, :-1]).logits
    assert torch.equal(full[:, 19:, :].argmax(-1), out[:, 20:])
    assert cuda_ops.device_status() == 0


@pytest.mark.parametrize("safe,dtype", [(True, torch.float32), (False, torch.float16)])
def test_checkpoint_round_trip_on_the_gpu(cuda_ops, tmp_path, safe, dtype):
    """save_pretrained -> from_pretrained(device="cuda") (the reference's inherited pair,
    benchmark/bench_opt.py:35-40): the reloaded model gives bit-identical logits and tokens."""
    from torch_int.models.opt import Int8OPTConfig, Int8OPTForCausalLM, Int8OPTModel
    from torch_int.models.random_init import random_int8_opt
    cfg = Int8OPTConfig(vocab_size=512, hidden_size=256, num_hidden_layers=3, ffn_dim=1024, num_attention_heads=4,
                        max_position_embeddings=256)
    model = random_int8_opt(cfg, seed=12, device="cuda", param_dtype=dtype)
    ids = torch.randint(0, cfg.vocab_size, (2, 77), generator=torch.Generator().manual_seed(2)).cuda()
    want = model(ids).logits
    model.save_pretrained(str(tmp_path), max_shard_bytes=300000, safe_serialization=safe)   # several files
    again = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cuda")
    assert next(again.parameters()).is_cuda and again.model.decoder.embed_tokens.weight.dtype == dtype
    assert_bit_exact(again(ids).logits.view(torch.int32 if dtype == torch.float32 else torch.int16),
                     want.view(torch.int32 if dtype == torch.float32 else torch.int16), "reloaded model")
    assert torch.equal(again.generate_greedy(ids[:, :30], 6), model.generate_greedy(ids[:, :30], 6))
    # the decoder-only class reads the same directory (keys with the "model." prefix)
    body = Int8OPTModel.from_pretrained(str(tmp_path), device="cuda")
    assert torch.equal(body(ids).last_hidden_state, model.model(ids).last_hidden_state)
    assert cuda_ops.device_status() == 0


def test_padding_mask(cuda_ops):
    cfg, model = small_model()
    sd = cpu_sd(model)
    g = torch.Generator().manual_seed(8)
    ids = torch.randint(2, cfg.vocab_size, (2, 48), generator=g)
    am = torch.ones((2, 48), dtype=torch.long)
    am[0, :9] = 0  # left padding on the first sequence
    ids[0, :9] = cfg.pad_token_id
    logits = model(ids.cuda(), attention_mask=am.cuda()).logits
    want, _ = OM.causal_lm_logits(sd, cfg, ids, am)
    keep = am.bool()
    assert rel_err(logits.cpu()[keep], want[keep]) < 2e-2


def test_static_cache_decode_matches_recompute(cuda_ops):
    """Prefill + token-by-token decoding with the static int8 cache gives the logits of a full
    forward over the same tokens (bit-exact: same kernels, same operands), and the oracle's tokens."""
    cfg, model = small_model()
    sd = cpu_sd(model)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab_size, (2, 21), generator=g)
    out = model.generate_greedy(prompt.cuda(), 6)
    assert out.shape == (2, 27) and torch.equal(out[:, :21].cpu(), prompt)
    full = model(out[:, :-1]).logits
    assert torch.equal(full[:, 20:, :].argmax(-1), out[:, 21:])
    cache = model.new_cache(2, 32)
    step_logits = [model(out[:, :21], past_key_values=cache, use_cache=True).logits[:, -1]]
    for t in range(21, 26):
        step_logits.append(model(out[:, t:t + 1], past_key_values=cache, use_cache=True).logits[:, -1])
    step_logits = torch.stack(step_logits, dim=1)
    assert rel_err(step_logits, full[:, 20:, :]) < 1e-6
    want, _ = OM.causal_lm_logits(sd, cfg, out[:, :-1].cpu())
    assert float((want[:, 20:, :].argmax(-1) == out[:, 21:].cpu()).double().mean()) >= 0.8
    assert cuda_ops.device_status() == 0


@pytest.mark.parametrize("bsz,heads,d,length", [(2, 3, 128, 0), (3, 2, 128, 37), (1, 4, 64, 200), (2, 2, 128, 1023)])
def test_decode_attention_kernel(cuda_ops, bsz, heads, d, length):
    """The one-token attention kernel against the op chain it replaces (bmm_s8t_s8n_f32t -> softmax ->
    x127 -> round -> bmm_s8t_s8n_s8t on the oracle), including the cache append at a device-side position."""
    C = cuda_ops
    e, cap = heads * d, 1024
    g = torch.Generator().manual_seed(3)
    keys = torch.randint(-127, 128, (bsz, cap, e), generator=g, dtype=torch.int8)
    vals = torch.randint(-127, 128, (bsz, heads, d, cap), generator=g, dtype=torch.int8)
    qkv = torch.randint(-60, 61, (bsz + 16, 3 * e), generator=g, dtype=torch.int8)
    a_qk, a_pv = 1.5 / (35.0 * 73.0 * d ** 0.5), 0.02
    kd, vd = keys.cuda(), vals.cuda()
    pos = torch.full((1,), length, dtype=torch.int32, device="cuda")
    ctx = C.decode_attention(qkv.cuda(), kd, vd, pos, a_qk, a_pv)
    # the cache received the new key row and value column
    assert torch.equal(kd[:, length].cpu(), qkv[:bsz, e:2 * e])
    assert torch.equal(vd[..., length].cpu(), qkv[:bsz, 2 * e:].view(bsz, heads, d))
    keys[:, length] = qkv[:bsz, e:2 * e]
    vals[..., length] = qkv[:bsz, 2 * e:].view(bsz, heads, d)
    assert torch.equal(kd.cpu(), keys) and torch.equal(vd.cpu(), vals), "nothing else in the cache may change"
    s = length + 1
    q = qkv[:bsz, :e].view(bsz, 1, heads, d).transpose(1, 2).reshape(bsz * heads, 1, d).contiguous()
    k = keys[:, :s].view(bsz, s, heads, d).transpose(1, 2).reshape(bsz * heads, s, d).contiguous()
    probs = O.softmax_q(O.bmm_s8t_s8n_f32t(q, k, a_qk))
    vt = vals[..., :s].reshape(bsz * heads, d, s).contiguous()
    want = O.bmm_s8t_s8n_s8t(probs, vt, a_pv).view(bsz, heads * d)
    # a probability that flips at a rounding tie moves a context value by up to alpha_pv * 127 = 2.5
    diff = (ctx.cpu().int() - want.int()).abs()
    assert int(diff.max()) <= 3 and float((diff == 0).double().mean()) >= 0.999, \
        (int(diff.max()), float((diff == 0).double().mean()))
    C.advance_position(pos, 1)
    assert int(pos.item()) == length + 1
    assert C.device_status() == 0


@pytest.mark.parametrize("bsz,heads,d,length", [(2, 2, 128, 127), (1, 3, 64, 500), (2, 1, 128, 1023)])
def test_decode_attention_probabilities(cuda_ops, bsz, heads, d, length):
    """The probabilities inside the one-token attention kernel, made visible: with alpha_pv = 1 and a value
    matrix that holds a single 1 per row (row r of head h selects position sel[h][r]), the context IS the
    int8 probability of the selected positions.  They obey the common rule of the softmax paths: at most
    one unit from the oracle, at least 99.9 % identical."""
    from helpers import assert_quant_close
    C = cuda_ops
    e, cap = heads * d, 1024
    s = length + 1
    g = torch.Generator().manual_seed(23)
    keys = torch.randint(-127, 128, (bsz, cap, e), generator=g, dtype=torch.int8)
    qkv = torch.randint(-60, 61, (bsz + 16, 3 * e), generator=g, dtype=torch.int8)
    a_qk = 1.5 / (35.0 * 73.0 * d ** 0.5)
    # the probabilities do not depend on the values: evaluate the oracle once
    kk = keys.clone()
    kk[:, length] = qkv[:bsz, e:2 * e]
    qh = qkv[:bsz, :e].view(bsz, 1, heads, d).transpose(1, 2).reshape(bsz * heads, 1, d).contiguous()
    kh = kk[:, :s].view(bsz, s, heads, d).transpose(1, 2).reshape(bsz * heads, s, d).contiguous()
    probs = O.softmax_q(O.bmm_s8t_s8n_f32t(qh, kh, a_qk)).view(bsz, heads, s)
    got, want = [], []
    for rep in range(4):                                  # different selections: 4 * d positions per head
        if rep == 0:    # the positions with the largest probabilities (of the first sequence), then random ones
            sel = torch.stack([probs[0, h].int().argsort(descending=True)[torch.arange(d) % s] for h in range(heads)])
        else:
            sel = torch.stack([torch.randperm(s, generator=g)[torch.arange(d) % s] for _ in range(heads)])
        vals = torch.zeros((bsz, heads, d, cap), dtype=torch.int8)
        for h in range(heads):
            vals[:, h, torch.arange(d), sel[h]] = 1
        # the kernel appends v of the new token at column `length`: make that column consistent with `vals`
        q3 = qkv.clone()
        q3[:bsz, 2 * e:] = vals[..., length].reshape(bsz, e)
        pos = torch.full((1,), length, dtype=torch.int32, device="cuda")
        ctx = C.decode_attention(q3.cuda(), keys.cuda(), vals.cuda(), pos, a_qk, 1.0).cpu().view(bsz, heads, d)
        got.append(ctx)
        want.append(torch.stack([probs[:, h, sel[h]] for h in range(heads)], dim=1))
    got, want = torch.cat(got), torch.cat(want)
    assert_quant_close(got, want, 0.999, "decode attention probabilities")
    assert int(want.int().abs().max()) >= 2               # the selection sees non-zero probabilities
    assert C.device_status() == 0


def test_decode_with_head_dim_80(cuda_ops):
    """Heads 80 wide (OPT-2.7B): neither one-kernel attention applies, prefill and decode steps take the
    three-kernel path, and decoding still reproduces the full forward."""
    cfg, model = small_model(layers=2, hidden=320, heads=4, ffn=640)
    assert model.model.decoder.layers[0].self_attn.head_dim == 80
    sd = cpu_sd(model)
    g = torch.Generator().manual_seed(14)
    prompt = torch.randint(0, cfg.vocab_size, (2, 19), generator=g)
    out = model.generate_greedy(prompt.cuda(), 5)
    full = model(out[:, :-1]).logits
    assert torch.equal(full[:, 18:, :].argmax(-1), out[:, 19:])
    want, _ = OM.causal_lm_logits(sd, cfg, out[:, :-1].cpu())
    assert rel_err(full, want) < 2e-2
    assert cuda_ops.device_status() == 0


def test_generate_with_and_without_cuda_graph(cuda_ops):
    cfg, model = small_model()
    g = torch.Generator().manual_seed(13)
    prompt = torch.randint(0, cfg.vocab_size, (3, 19), generator=g).cuda()
    eager = model.generate_greedy(prompt, 12, use_cuda_graph=False)
    cache = model.new_cache(3, 64)
    graphed = model.generate_greedy(prompt, 12, cache=cache, use_cuda_graph=True)
    again = model.generate_greedy(prompt, 12, cache=cache, use_cuda_graph=True)  # replays the stored graph
    assert torch.equal(eager, graphed) and torch.equal(graphed, again)
    assert cache.length == 19 + 11 and int(cache.pos.item()) == cache.length
    assert cuda_ops.device_status() == 0
