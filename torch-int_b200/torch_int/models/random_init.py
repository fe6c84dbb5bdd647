"""Seeded random Int8 OPT models for benchmarks and tests.

No OPT checkpoint is needed: int8 weights are uniform on [-127, 127], LayerNorm
gains ~ N(1, 0.1) x g and shifts ~ N(0, 0.1) x g, and the per-tensor scales are
the analytic values that keep every int8 activation at a standard deviation of a
few tens (so results neither saturate nor collapse to zero), each multiplied by
a seeded factor ~ U(0.7, 1.3).
"""
import math
import zlib

import torch

from .opt import Int8OPTConfig, Int8OPTForCausalLM
from .tensor_parallel import TensorParallel

SIGMA_W = 127.0 / math.sqrt(3.0)  # standard deviation of uniform int8 weights
ACT_SIGMA = 30.0                  # target standard deviation of int8 activations


def analytic_scales(hidden, ffn, head_dim):
    """alpha of every op for int8 activations of standard deviation ACT_SIGMA."""
    s = ACT_SIGMA
    return {
        "qkv": s / (s * SIGMA_W * math.sqrt(hidden)),
        "qk": 1.5 / (s * s * math.sqrt(head_dim)),
        "pv": 0.05,
        "out": 0.3 / (10.0 * SIGMA_W * math.sqrt(hidden)),
        "fc1": 40.0 / (s * SIGMA_W * math.sqrt(hidden)),
        "fc2": 0.3 / (25.0 * SIGMA_W * math.sqrt(ffn)),
    }


def _cpu_gen(seed, *tags):
    g = torch.Generator()
    # a process-independent key (Python's hash() of strings is salted per process)
    g.manual_seed(zlib.crc32(repr((seed,) + tags).encode()))
    return g


@torch.no_grad()
def init_random_(model: Int8OPTForCausalLM, seed: int = 0, consistent: bool = True):
    """Fills `model` in place.  consistent=True draws every FULL tensor from a CPU
    generator keyed by (seed, layer, name) and keeps this rank's slice, so all
    tensor-parallel layouts hold the same model; consistent=False draws each rank's
    slice of the split int8 weights directly on its device (fast, for large benchmark models).
    The replicated parameters (scales, LayerNorm, fp32 biases, embeddings) depend on `seed` alone
    in both modes: ranks that pass the same seed hold one coherent model."""
    dec = model.model.decoder
    cfg, tp = model.config, dec.tp
    dev = dec.embed_tokens.weight.device
    e, f, heads = cfg.hidden_size, cfg.ffn_dim, cfg.num_attention_heads
    sc = analytic_scales(e, f, e // heads)

    def jitter(li, name):
        return float(0.7 + 0.6 * torch.rand((), generator=_cpu_gen(seed, li, name, "jitter")))

    # consistent=False: this rank's slices come from a device generator keyed by (seed, rank), so that
    # a run is reproducible and the ranks hold different slices of one model
    dev_gen = None
    if not consistent and torch.device(dev).type == "cuda":
        dev_gen = torch.Generator(device=dev)
        dev_gen.manual_seed(zlib.crc32(repr((seed, "slices", tp.rank)).encode()))

    def s8(shape_full, li, name, kind):
        """kind: 'rows' (column-parallel weight), 'cols' (row-parallel weight), 'vec' ([1,N] bias of a
        column-parallel linear) or 'full'."""
        if consistent:
            t = torch.randint(-127, 128, shape_full, generator=_cpu_gen(seed, li, name), dtype=torch.int8)
            if kind == "rows":
                t = tp._rows(t)
            elif kind == "cols" or kind == "vec":
                t = tp._cols(t)
            return t.to(dev)
        shape = list(shape_full)
        if kind == "rows":
            shape[0] //= tp.size
        elif kind in ("cols", "vec"):
            shape[-1] //= tp.size
        return torch.randint(-127, 128, shape, dtype=torch.int8, device=dev, generator=dev_gen)

    def f32(shape, li, name, std, mean=0.0):
        t = torch.randn(shape, generator=_cpu_gen(seed, li, name)) * std + mean
        return t.to(dev)

    for li, layer in enumerate(dec.layers):
        a = layer.self_attn
        for name, lin in (("q_proj", a.q_proj), ("k_proj", a.k_proj), ("v_proj", a.v_proj)):
            lin.weight = s8((e, e), li, name + ".w", "rows")
            lin.bias = s8((1, e), li, name + ".b", "vec")
            lin.a = torch.tensor(sc["qkv"] * jitter(li, name), device=dev)
            lin.b = torch.tensor(0.05, device=dev)
        a.qk_bmm.a = torch.tensor(sc["qk"] * jitter(li, "qk"), device=dev)
        a.pv_bmm.a = torch.tensor(sc["pv"] * jitter(li, "pv"), device=dev)
        a.out_proj.weight = s8((e, e), li, "out_proj.w", "cols")
        a.out_proj.bias = f32((1, e), li, "out_proj.b", 0.02)
        a.out_proj.a = torch.tensor(sc["out"] * jitter(li, "out"), device=dev)
        layer.fc1.weight = s8((f, e), li, "fc1.w", "rows")
        layer.fc1.bias = s8((1, f), li, "fc1.b", "vec")
        layer.fc1.a = torch.tensor(sc["fc1"] * jitter(li, "fc1"), device=dev)
        layer.fc1.b = torch.tensor(0.05, device=dev)
        layer.fc2.weight = s8((e, f), li, "fc2.w", "cols")
        layer.fc2.bias = f32((1, e), li, "fc2.b", 0.02)
        layer.fc2.a = torch.tensor(sc["fc2"] * jitter(li, "fc2"), device=dev)
        for name, ln in (("ln1", layer.self_attn_layer_norm), ("ln2", layer.final_layer_norm)):
            ln.weight = f32((e,), li, name + ".w", 0.1 * ACT_SIGMA, ACT_SIGMA)
            ln.bias = f32((e,), li, name + ".b", 0.1 * ACT_SIGMA)
    wdtype = dec.embed_tokens.weight.dtype
    dec.embed_tokens.weight.copy_(f32(tuple(dec.embed_tokens.weight.shape), -1, "embed", 0.7).to(wdtype))
    dec.embed_positions.weight.copy_(f32(tuple(dec.embed_positions.weight.shape), -1, "pos", 0.3).to(wdtype))
    if dec.final_layer_norm is not None:
        dec.final_layer_norm.weight.copy_(f32((e,), -1, "final_ln.w", 0.1, 1.0).to(wdtype))
        dec.final_layer_norm.bias.copy_(f32((e,), -1, "final_ln.b", 0.1).to(wdtype))
    return model


def random_int8_opt(config: Int8OPTConfig, seed: int = 0, device="cuda", tp: TensorParallel = None,
                    param_dtype=torch.float32, consistent: bool = True) -> Int8OPTForCausalLM:
    """Builds a random Int8OPTForCausalLM on `device` (embeddings / lm_head / final
    LayerNorm in `param_dtype`)."""
    with torch.device(device):
        model = Int8OPTForCausalLM(config, tp=tp)
    model.model.decoder.embed_tokens.to(param_dtype)
    model.model.decoder.embed_positions.to(param_dtype)
    if model.model.decoder.final_layer_norm is not None:
        model.model.decoder.final_layer_norm.to(param_dtype)
    model.lm_head.weight = model.model.decoder.embed_tokens.weight
    init_random_(model, seed, consistent)
    return model.eval()


OPT_ARCHS = {
    # hidden, layers, heads, ffn  (vocab 50272, 2048 positions)
    "opt-125m": (768, 12, 12, 3072),
    "opt-1.3b": (2048, 24, 32, 8192),
    "opt-6.7b": (4096, 32, 32, 16384),
    "opt-13b": (5120, 40, 40, 20480),
    "opt-30b": (7168, 48, 56, 28672),
    "opt-66b": (9216, 64, 72, 36864),
    "opt-175b": (12288, 96, 96, 49152),
}


def opt_config(name: str, **overrides) -> Int8OPTConfig:
    h, l, a, f = OPT_ARCHS[name]
    return Int8OPTConfig(vocab_size=50272, hidden_size=h, num_hidden_layers=l, ffn_dim=f,
                         num_attention_heads=a, max_position_embeddings=2048, **overrides)
