"""Host logic of torch_int.models.opt on CPU: the model's own Python (views and strides handed to the strided
GEMM, the static cache, masks, the fused residual/LayerNorm order, decoding) runs with the extension module
replaced by oracle-backed stand-ins (tests/cpu_ops_stub.py) and must reproduce the oracle's restatement of
the REFERENCE model dataflow (oracle/opt_model.py) bit for bit.  The kernels themselves are covered by the
-m gpu tests; this file keeps the wiring honest where no GPU is available."""
import pytest
import torch

import cpu_ops_stub as stub
from oracle import opt_model as OM


@pytest.fixture()
def cpu_model(monkeypatch):
    from torch_int.models.opt import Int8OPTConfig
    from torch_int.models.random_init import random_int8_opt
    stub.install(monkeypatch.setattr)
    cfg = Int8OPTConfig(vocab_size=96, hidden_size=128, num_hidden_layers=2, ffn_dim=256, num_attention_heads=2,
                        max_position_embeddings=64)
    model = random_int8_opt(cfg, seed=7, device="cpu")
    sd = {k: v.detach().clone() for k, v in model.state_dict().items()}
    return model, cfg, sd


def ids(b, t, seed):
    return torch.randint(2, 96, (b, t), generator=torch.Generator().manual_seed(seed))


def test_fused_wiring_equals_the_reference_dataflow(cpu_model):
    model, cfg, sd = cpu_model
    x = ids(2, 21, 1)                      # 21: not a multiple of 16, the key length is padded inside attention
    want, _ = OM.causal_lm_logits(sd, cfg, x)
    got = model(x).logits
    assert got.shape == want.shape and torch.equal(got, want)
    # (a one-row lm_head product may round differently from the batched one in the CPU BLAS)
    assert torch.allclose(model(x, last_token_only=True).logits, want[:, -1:], rtol=1e-5, atol=1e-5)
    # the reference-signature modules (they need a key length that is a multiple of 16, as the reference does)
    x = ids(2, 32, 5)
    want, _ = OM.causal_lm_logits(sd, cfg, x)
    assert torch.equal(model(x, reference_path=True).logits, want)
    assert torch.equal(model(x).logits, want)


def test_padding_mask(cpu_model):
    model, cfg, sd = cpu_model
    x = ids(2, 18, 2)
    mask = torch.ones(2, 18, dtype=torch.long)
    mask[1, :5] = 0                        # left padding of the second sequence
    want, _ = OM.causal_lm_logits(sd, cfg, x, attention_mask=mask)
    got = model(x, attention_mask=mask).logits
    assert torch.equal(got[0], want[0]) and torch.equal(got[1, 5:], want[1, 5:])


def test_fused_attention_switch_keeps_the_result(cpu_model):
    model, cfg, sd = cpu_model
    x = ids(2, 33, 3)
    base = model(x).logits
    for layer in model.model.decoder.layers:
        layer.self_attn.fused_attention = True
    assert torch.equal(model(x).logits, base)
    # with a cache as well (keys and transposed values come from the cache views)
    cache = model.new_cache(2, 48)
    assert torch.equal(model(x, past_key_values=cache, use_cache=True).logits, base)


def test_static_cache_prefill_and_decode_steps(cpu_model):
    model, cfg, sd = cpu_model
    x = ids(2, 12, 4)
    steps = 5
    out = model.generate_greedy(x, steps, use_cuda_graph=False)
    assert out.shape == (2, 12 + steps) and torch.equal(out[:, :12], x)
    # teacher forcing: the full forward over the generated sequence predicts the same tokens, and the
    # logits of a decode step equal the full forward's logits at that position
    full = model(out[:, :-1]).logits
    assert torch.equal(full[:, 11:].argmax(-1), out[:, 12:])
    cache = model.new_cache(2, 32)
    model(out[:, :14], past_key_values=cache, use_cache=True)
    dec = model.model.decoder
    want = dec(out[:, :15]).last_hidden_state[:, -1]          # hidden state before the lm_head: exact
    step_hidden = dec.decode_step(out[:, 14:15], cache)
    assert cache.length == 15
    assert torch.equal(step_hidden[:, -1], want)
    # chunked prefill through the cache: 9 tokens, then 6 more
    cache2 = model.new_cache(2, 32)
    model(out[:, :9], past_key_values=cache2, use_cache=True)
    second = dec(out[:, 9:15], past_key_values=cache2, use_cache=True).last_hidden_state
    assert torch.equal(second[:, -1], want)
    with pytest.raises(RuntimeError, match="capacity"):
        model.generate_greedy(x, 30, cache=cache2)
