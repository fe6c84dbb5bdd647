"""Checkpoint directories in the transformers layout (config.json + state-dict files with the reference's
buffer names): save -> load round trips, the file variants the reference's tools produce, and per-rank
slice loading for tensor parallelism.  CPU only: models are built and filled, never run."""
import json
import os

import pytest
import torch

from torch_int.models import checkpoint as ckpt
from torch_int.models.opt import Int8OPTConfig, Int8OPTForCausalLM, Int8OPTModel
from torch_int.models.random_init import random_int8_opt
from torch_int.models.tensor_parallel import TensorParallel

CFG = dict(vocab_size=96, hidden_size=64, num_hidden_layers=3, ffn_dim=128, num_attention_heads=4,
           max_position_embeddings=32)


def small_model(seed=3, dtype=torch.float32):
    return random_int8_opt(Int8OPTConfig(**CFG), seed=seed, device="cpu", param_dtype=dtype)


def same_state(a, b):
    assert a.keys() == b.keys(), sorted(set(a) ^ set(b))[:5]
    for k in a:
        assert a[k].dtype == b[k].dtype and a[k].shape == b[k].shape, (k, a[k].dtype, b[k].dtype, a[k].shape, b[k].shape)
        assert torch.equal(a[k], b[k]), k


@pytest.mark.parametrize("safe", [True, False])
@pytest.mark.parametrize("shard_bytes", [5 << 30, 20000])
def test_round_trip(tmp_path, safe, shard_bytes):
    model = small_model()
    files = model.save_pretrained(str(tmp_path), max_shard_bytes=shard_bytes, safe_serialization=safe)
    if shard_bytes < 1 << 20:
        assert len(files) > 2
        index = "model.safetensors.index.json" if safe else "pytorch_model.bin.index.json"
        weight_map = json.load(open(tmp_path / index))["weight_map"]
        assert set(weight_map.values()) == set(files) and "lm_head.weight" not in weight_map
    else:
        assert files == ["model.safetensors" if safe else "pytorch_model.bin"]
    conf = json.load(open(tmp_path / "config.json"))
    assert conf["model_type"] == "opt" and conf["hidden_size"] == 64 and conf["torch_dtype"] == "float32"
    again = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    same_state(model.state_dict(), again.state_dict())
    assert again.lm_head.weight is again.model.decoder.embed_tokens.weight
    # saving again with another split leaves no stale files behind
    model.save_pretrained(str(tmp_path), safe_serialization=safe)
    assert sorted(os.listdir(tmp_path)) == sorted(["config.json", "model.safetensors" if safe else "pytorch_model.bin"])


def test_fused_qkv_views_are_saved_compactly(tmp_path):
    model = small_model()
    before = {k: v.clone() for k, v in model.state_dict().items()}
    for layer in model.model.decoder.layers:      # what the first forward does: q/k/v become views of one tensor
        layer.self_attn._fused_qkv()
    model.save_pretrained(str(tmp_path))
    assert os.path.getsize(tmp_path / "model.safetensors") < 1.2 * sum(
        v.numel() * v.element_size() for k, v in before.items() if k != "lm_head.weight") + 20000
    same_state(before, Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu").state_dict())


@pytest.mark.parametrize("size", [2, 4])
@pytest.mark.parametrize("safe", [True, False])
def test_each_rank_loads_its_slices(tmp_path, size, safe):
    model = small_model()
    model.save_pretrained(str(tmp_path), max_shard_bytes=30000, safe_serialization=safe)
    full = model.state_dict()
    for rank in range(size):
        tp = TensorParallel(size, rank)
        part = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu", tp=tp)
        same_state(tp.shard_state_dict(full), part.state_dict())
        attn = part.model.decoder.layers[0].self_attn
        assert attn.q_proj.weight.shape == (64 // size, 64) and attn.out_proj.weight.shape == (64, 64 // size)


def test_reference_file_variants(tmp_path):
    """[N] int8 biases and 1-element scales (what from_float leaves behind), `decoder.*` keys of an
    Int8OPTModel checkpoint, and a pytorch_model.bin: all load into Int8OPTForCausalLM."""
    model = small_model()
    state = {}
    for k, v in model.model.state_dict().items():          # keys: decoder.*
        if k.endswith("_proj.bias") or k.endswith("fc1.bias") or k.endswith("fc2.bias"):
            v = v.reshape(-1)
        elif v.dim() == 0:
            v = v.reshape(1)
        state[k] = v.clone()
    torch.save(state, tmp_path / "pytorch_model.bin")
    json.dump(dict(CFG, model_type="opt", torch_dtype="float32"), open(tmp_path / "config.json", "w"))
    again = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu", device_map="auto")
    same_state(model.state_dict(), again.state_dict())
    bare = Int8OPTModel.from_pretrained(str(tmp_path), device="cpu")
    same_state(model.model.state_dict(), bare.state_dict())
    # ... and a causal-LM checkpoint into the bare model
    model.save_pretrained(str(tmp_path / "lm"), safe_serialization=False)
    same_state(model.model.state_dict(), Int8OPTModel.from_pretrained(str(tmp_path / "lm"), device="cpu").state_dict())


def test_float_dtype(tmp_path):
    model = small_model(dtype=torch.float16)
    model.save_pretrained(str(tmp_path))
    assert json.load(open(tmp_path / "config.json"))["torch_dtype"] == "float16"
    again = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    dec = again.model.decoder
    assert dec.embed_tokens.weight.dtype == torch.float16 and dec.final_layer_norm.weight.dtype == torch.float16
    assert dec.layers[0].fc1.weight.dtype == torch.int8 and dec.layers[0].fc1.a.dtype == torch.float32
    assert dec.layers[0].self_attn_layer_norm.weight.dtype == torch.float32
    same_state(model.state_dict(), again.state_dict())
    wide = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu", torch_dtype=torch.float32)
    assert wide.model.decoder.embed_tokens.weight.dtype == torch.float32
    assert torch.equal(wide.model.decoder.embed_tokens.weight, dec.embed_tokens.weight.float())


def test_errors(tmp_path):
    with pytest.raises(FileNotFoundError):
        Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    model = small_model()
    model.save_pretrained(str(tmp_path), safe_serialization=False)
    state = torch.load(tmp_path / "pytorch_model.bin")
    # a missing tensor
    broken = {k: v for k, v in state.items() if not k.endswith("layers.1.fc2.weight")}
    torch.save(broken, tmp_path / "pytorch_model.bin")
    with pytest.raises(KeyError, match="fc2.weight"):
        Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    missing, unexpected = ckpt.load_into(small_model(seed=9), str(tmp_path), strict=False)
    assert missing == ["model.decoder.layers.1.fc2.weight"] and unexpected == []
    # an unknown tensor
    torch.save(dict(state, **{"model.decoder.layers.0.rotary.inv_freq": torch.zeros(4)}), tmp_path / "pytorch_model.bin")
    with pytest.raises(KeyError, match="inv_freq"):
        Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    # a wrong shape and a wrong dtype
    k = "model.decoder.layers.0.fc1.weight"
    torch.save(dict(state, **{k: state[k][:, :32].contiguous()}), tmp_path / "pytorch_model.bin")
    with pytest.raises(ValueError, match="fc1.weight"):
        Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    torch.save(dict(state, **{k: state[k].float()}), tmp_path / "pytorch_model.bin")
    with pytest.raises(ValueError, match="dtype"):
        Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu")
    # heads that do not divide over the ranks
    torch.save(state, tmp_path / "pytorch_model.bin")
    with pytest.raises(ValueError):
        Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu", tp=TensorParallel(3, 0))
    # a split model cannot be written as a whole one
    part = Int8OPTForCausalLM.from_pretrained(str(tmp_path), device="cpu", tp=TensorParallel(2, 1))
    with pytest.raises(RuntimeError, match="rank 1 of 2"):
        part.save_pretrained(str(tmp_path / "part"))


@pytest.mark.parametrize("safe", [True, False])
def test_per_rank_checkpoints(tmp_path, safe):
    model = small_model()
    model.save_pretrained(str(tmp_path / "whole"), max_shard_bytes=40000, safe_serialization=safe)
    dirs = ckpt.write_rank_shards(str(tmp_path / "whole"), str(tmp_path / "split"), 2, max_shard_bytes=25000,
                                  safe_serialization=safe)
    assert dirs == [ckpt.rank_directory(str(tmp_path / "split"), 2, r) for r in range(2)]
    full = model.state_dict()
    for rank, d in enumerate(dirs):
        assert json.load(open(os.path.join(d, "config.json")))["tensor_parallel"] == {"size": 2, "rank": rank}
        tp = TensorParallel(2, rank)
        part = Int8OPTForCausalLM.from_pretrained(d, device="cpu", tp=tp)
        same_state(tp.shard_state_dict(full), part.state_dict())
    with pytest.raises(ValueError, match="holds rank 1 of 2"):
        Int8OPTForCausalLM.from_pretrained(dirs[1], device="cpu", tp=TensorParallel(2, 0))
    with pytest.raises(ValueError, match="holds rank 0 of 2"):
        Int8OPTForCausalLM.from_pretrained(dirs[0], device="cpu")
    with pytest.raises(ValueError, match="already a per-rank"):
        ckpt.write_rank_shards(dirs[0], str(tmp_path / "again"), 2)
