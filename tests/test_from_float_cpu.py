"""`from_float` conversion of float OPT modules (transformers) into the Int8 OPT modules, evaluated
on CPU with the oracle: the analogue of the reference's tests/test_opt_decoder_layer.py and
tests/test_opt_decoder.py (which print an r2 error of the int8 model against the float model), with
random-init float models instead of downloaded checkpoints and with thresholds."""
import pytest
import torch

from oracle import opt_model as OM
from oracle import w8a8 as O

transformers = pytest.importorskip("transformers")
from transformers.models.opt.modeling_opt import OPTConfig, OPTDecoderLayer, OPTForCausalLM  # noqa: E402


def _config(layers=2):
    cfg = OPTConfig(hidden_size=128, num_attention_heads=4, ffn_dim=512, num_hidden_layers=layers, vocab_size=256,
                    max_position_embeddings=128, word_embed_proj_dim=128)
    cfg._attn_implementation = "eager"
    return cfg


def _calibrate(layer, run):
    """absmax / 127 of the seven activations Int8OPTDecoderLayer.from_float needs, collected with
    forward hooks as tests/test_opt_decoder_layer.py:28-40 of the reference does."""
    stats = {}

    def hook(name, pick_input):
        def fn(mod, inp, out):
            t = inp[0] if pick_input else out
            stats[name] = max(stats.get(name, 0.0), float(t.detach().abs().max()))
        return fn

    a = layer.self_attn
    handles = [layer.self_attn_layer_norm.register_forward_hook(hook("attn_input_scale", False)),
               a.q_proj.register_forward_hook(hook("q_output_scale", False)),
               a.k_proj.register_forward_hook(hook("k_output_scale", False)),
               a.v_proj.register_forward_hook(hook("v_output_scale", False)),
               a.out_proj.register_forward_hook(hook("out_input_scale", True)),
               layer.fc1.register_forward_hook(hook("fc1_input_scale", True)),
               layer.fc2.register_forward_hook(hook("fc2_input_scale", True))]
    with torch.no_grad():
        run()
    for h in handles:
        h.remove()
    return {k: v / 127.0 for k, v in stats.items()}


def _r2(got, want):
    return float(((got.double() - want.double()) ** 2).mean() / (want.double() ** 2).mean())


def test_decoder_layer_from_float():
    from torch_int.models.opt import Int8OPTDecoderLayer
    torch.manual_seed(0)
    layer = OPTDecoderLayer(_config(), layer_idx=0).eval()
    for p in layer.parameters():  # away from the near-zero default init so that scales are meaningful
        p.data.normal_(0, 0.05) if p.dim() > 1 else p.data.normal_(0, 0.02)
    layer.self_attn_layer_norm.weight.data.fill_(1.0)
    layer.final_layer_norm.weight.data.fill_(1.0)
    before = {k: v.clone() for k, v in layer.state_dict().items()}
    x = torch.randn(2, 32, 128)
    mask = O.causal_mask(2, 32, 32)
    scales = _calibrate(layer, lambda: layer(x, attention_mask=mask))
    int8_layer = Int8OPTDecoderLayer.from_float(layer, **scales)
    assert all(torch.equal(v, before[k]) for k, v in layer.state_dict().items()), "from_float must not modify the float layer"
    a = int8_layer.self_attn
    # scale folding of torch_int/models/opt.py:61-77 and torch_int/nn/linear.py:46-57
    scaling = layer.self_attn.scaling
    wq = layer.self_attn.q_proj.weight.detach() * scaling
    assert torch.allclose(a.q_proj.a, scales["attn_input_scale"] * (wq.abs().max() / 127) / (scales["q_output_scale"] * scaling))
    assert abs(float(a.qk_bmm.a) - scales["q_output_scale"] * scaling * scales["k_output_scale"]) < 1e-9
    assert abs(float(a.pv_bmm.a) - (1.0 / 127) * scales["v_output_scale"] / scales["out_input_scale"]) < 1e-9
    assert torch.allclose(int8_layer.self_attn_layer_norm.weight, layer.self_attn_layer_norm.weight / scales["attn_input_scale"])
    sd = {f"L.{k}": v.detach() for k, v in int8_layer.state_dict().items()}
    with torch.no_grad():
        want = layer(x, attention_mask=mask)
        want = want[0] if isinstance(want, tuple) else want
    got, _ = OM.decoder_layer(sd, "L", x, mask, 4)
    assert _r2(got, want) < 0.02, _r2(got, want)


def test_causal_lm_from_float():
    from torch_int.models.opt import Int8OPTForCausalLM
    torch.manual_seed(1)
    cfg = _config(layers=2)
    model = OPTForCausalLM(cfg).eval()
    for n, p in model.named_parameters():
        if p.dim() > 1 and "embed" not in n:
            p.data.normal_(0, 0.05)
    ids = torch.randint(2, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(2))
    layers = model.model.decoder.layers
    all_scales = [None] * len(layers)
    for i, layer in enumerate(layers):
        all_scales[i] = _calibrate(layer, lambda: model(ids))
    int8_model = Int8OPTForCausalLM.from_float(model, all_scales)
    sd = {k: v.detach() for k, v in int8_model.state_dict().items()}
    assert "model.decoder.layers.1.fc2.weight" in sd and sd["model.decoder.layers.0.self_attn.q_proj.weight"].dtype == torch.int8
    with torch.no_grad():
        want = model(ids).logits
    got, _ = OM.causal_lm_logits(sd, cfg, ids)
    assert got.shape == want.shape
    assert _r2(got, want) < 0.05, _r2(got, want)
    assert float((got.argmax(-1) == want.argmax(-1)).double().mean()) > 0.8


def test_converted_model_runs_through_the_product_wiring(monkeypatch):
    """The modules as from_float leaves them ([N] int8 biases, scales as tensors or Python floats, the float
    model's embedding modules) go through the product's own forward - fused q/k/v weights, strided attention,
    fused residual/LayerNorm steps - with the extension replaced by oracle-backed stand-ins, and give exactly
    the oracle's reference dataflow on the converted state dict."""
    import cpu_ops_stub as stub
    from torch_int.models.opt import Int8OPTForCausalLM
    torch.manual_seed(3)
    cfg = _config(layers=2)
    model = OPTForCausalLM(cfg).eval()
    ids = torch.randint(2, cfg.vocab_size, (2, 19), generator=torch.Generator().manual_seed(4))
    scales = [_calibrate(layer, lambda: model(ids)) for layer in model.model.decoder.layers]
    int8_model = Int8OPTForCausalLM.from_float(model, scales)
    sd = {k: v.detach().clone() for k, v in int8_model.state_dict().items()}
    stub.install(monkeypatch.setattr)
    want, _ = OM.causal_lm_logits(sd, cfg, ids)
    got = int8_model(ids).logits
    assert torch.equal(got, want)
    cache = int8_model.new_cache(2, 32)
    assert torch.equal(int8_model(ids, past_key_values=cache, use_cache=True).logits, want)


def test_from_float_model_saves_and_loads(tmp_path):
    """A quantised model as from_float leaves it (transformers' config object, the float embedding modules
    of the source model) goes through save_pretrained / from_pretrained unchanged."""
    from torch_int.models.opt import Int8OPTForCausalLM
    torch.manual_seed(4)
    cfg = _config(layers=1)
    model = OPTForCausalLM(cfg).eval()
    scales = [dict(attn_input_scale=0.05, q_output_scale=0.04, k_output_scale=0.04, v_output_scale=0.03,
                   out_input_scale=0.02, fc1_input_scale=0.05, fc2_input_scale=0.03)]
    int8_model = Int8OPTForCausalLM.from_float(model, scales)
    int8_model.save_pretrained(str(tmp_path))
    again = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    a, b = int8_model.state_dict(), again.state_dict()
    assert set(a) == set(b)
    for k in a:
        assert torch.equal(a[k].reshape(-1).float(), b[k].reshape(-1).float()), k
