"""Int8 OPT attention / decoder layer / causal LM on the GPU against the CPU
restatement of the reference's dataflow (oracle/opt_model.py)."""
import pytest
import torch

from helpers import assert_bit_exact, rand_s8, randn, set_fused_attention
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
    diff = (ctx.cpu().int() - want.int()).abs()
    assert int(diff.max()) <= 2 and float((diff == 0).double().mean()) > 0.97, (int(diff.max()), float((diff == 0).double().mean()))
    C.advance_position(pos, 1)
    assert int(pos.item()) == length + 1
    assert C.device_status() == 0


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
