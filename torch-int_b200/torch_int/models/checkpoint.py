"""Reading and writing Int8 OPT checkpoints.

The reference's Int8 OPT classes inherit transformers' OPTPreTrainedModel
(torch_int/models/opt.py:302,401,420), so its checkpoints are whatever
``save_pretrained`` / ``from_pretrained`` of transformers produce and read
(benchmark/bench_opt.py:24-40): a directory with

  config.json                                     the OPTConfig fields
  pytorch_model.bin | model.safetensors           one state dict, or
  pytorch_model-0000i-of-0000n.bin + pytorch_model.bin.index.json   (sharded)
  model-0000i-of-0000n.safetensors + model.safetensors.index.json   (sharded)

with the reference's buffer names (``model.decoder.layers.3.fc1.weight`` int8,
``...fc1.a`` fp32 scalar, ...).  The classes here do not inherit from
transformers, so this module restates that directory format:

* ``load_pretrained`` builds the model directly on the target device and fills
  it tensor by tensor.  With a ``TensorParallel`` context every rank reads only
  its own rows / columns of the split weights from the files (safetensors slices,
  or pages of a memory-mapped ``.bin``): an OPT-175B checkpoint is read once in
  total, not once per rank, and no rank ever holds a whole weight matrix.
* ``save_pretrained`` writes the same layout (single-GPU models).

Accepted variations of the files the reference's own tools produce: int8 linear
biases stored as [N] (after ``from_float``, nn/linear.py:54) or [1, N] (as
constructed, nn/linear.py:25-26); scales stored as 0-d or 1-element tensors; keys
with or without the ``model.`` prefix (``Int8OPTModel`` vs ``Int8OPTForCausalLM``
checkpoints); ``lm_head.weight`` absent (it is tied to the token embedding).
"""
import json
import os
import re
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .tensor_parallel import TensorParallel

CONFIG_NAME = "config.json"
_BIN, _BIN_INDEX = "pytorch_model.bin", "pytorch_model.bin.index.json"
_ST, _ST_INDEX = "model.safetensors", "model.safetensors.index.json"
_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
           "float": torch.float32, "half": torch.float16}


# --------------------------------------------------------------------------- config.json
def _config_fields():
    from .opt import Int8OPTConfig
    import dataclasses
    return [f.name for f in dataclasses.fields(Int8OPTConfig)]


def read_config(directory: str):
    """The Int8OPTConfig of a checkpoint directory and the float dtype its config.json names (or None)."""
    from .opt import Int8OPTConfig
    path = os.path.join(directory, CONFIG_NAME)
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{path}: a checkpoint directory needs a config.json")
    with open(path) as f:
        raw = json.load(f)
    kw = {k: raw[k] for k in _config_fields() if k in raw}
    for required in ("hidden_size", "num_hidden_layers", "num_attention_heads", "ffn_dim", "vocab_size"):
        if required not in kw:
            raise ValueError(f"{path}: missing field {required!r}")
    name = raw.get("torch_dtype", raw.get("dtype"))
    return Int8OPTConfig(**kw), _DTYPES.get(str(name).replace("torch.", "")) if name else None


def config_dict(config, float_dtype: torch.dtype, architecture: str) -> dict:
    out = {"model_type": "opt", "architectures": [architecture]}
    for k in _config_fields():
        if hasattr(config, k):
            out[k] = getattr(config, k)
    out["torch_dtype"] = str(float_dtype).replace("torch.", "")
    return out


# --------------------------------------------------------------------------- tensor sources
class _Source:
    """One tensor inside a checkpoint file: its shape, and reading all or a slice of it."""

    def __init__(self, shape, itemsize, read):
        self.shape = tuple(shape)
        self.itemsize = itemsize
        self._read = read

    def read(self, dim: Optional[int] = None, start: int = 0, stop: Optional[int] = None) -> torch.Tensor:
        if dim is None or len(self.shape) == 0:
            return self._read(None)
        dim = dim % len(self.shape)
        index = tuple(slice(start, stop) if d == dim else slice(None) for d in range(len(self.shape)))
        return self._read(index)


class _Files:
    """The tensor files of a checkpoint directory, opened lazily and kept open while loading."""

    def __init__(self, directory: str):
        self.directory = directory
        self._open: Dict[str, object] = {}
        self.names: Dict[str, str] = {}      # tensor name -> file name
        listing = set(os.listdir(directory))
        if _ST_INDEX in listing or _BIN_INDEX in listing:
            index = _ST_INDEX if _ST_INDEX in listing else _BIN_INDEX
            with open(os.path.join(directory, index)) as f:
                self.names = dict(json.load(f)["weight_map"])
            missing = sorted(set(self.names.values()) - listing)
            if missing:
                raise FileNotFoundError(f"{directory}: {index} names files that are absent: {missing[:3]}")
        elif _ST in listing or _BIN in listing:
            fname = _ST if _ST in listing else _BIN
            self.names = {name: fname for name in self._tensor_names(fname)}
        else:
            raise FileNotFoundError(f"{directory}: no {_ST}, {_BIN} or sharded index found")

    def _handle(self, fname):
        h = self._open.get(fname)
        if h is None:
            path = os.path.join(self.directory, fname)
            if fname.endswith(".safetensors"):
                from safetensors import safe_open
                h = safe_open(path, framework="pt", device="cpu")
            else:
                try:      # memory-mapped: a slice touches only its own pages of the file
                    h = torch.load(path, map_location="cpu", mmap=True, weights_only=True)
                except (RuntimeError, ValueError):   # files written in the pre-zip format cannot be mapped
                    h = torch.load(path, map_location="cpu", weights_only=True)
                if not isinstance(h, dict):
                    raise ValueError(f"{path}: expected a state dict, found {type(h).__name__}")
            self._open[fname] = h
        return h

    def _tensor_names(self, fname) -> Iterable[str]:
        return list(self._handle(fname).keys())

    def source(self, name: str) -> _Source:
        fname = self.names[name]
        h = self._handle(fname)
        if fname.endswith(".safetensors"):
            sl = h.get_slice(name)
            bits = re.search(r"\d+", sl.get_dtype())       # "I8", "F32", "BF16", ...; "BOOL" is one byte
            return _Source(sl.get_shape(), int(bits.group()) // 8 if bits else 1,
                           lambda idx, sl=sl, h=h, name=name: h.get_tensor(name) if idx is None else sl[idx])
        t = h[name]
        return _Source(t.shape, t.element_size(), lambda idx, t=t: t if idx is None else t[idx])

    def close(self):
        self._open.clear()


# --------------------------------------------------------------------------- loading
def _target_name(key: str, targets: Dict[str, torch.Tensor]) -> Optional[str]:
    """Checkpoint key -> model key: Int8OPTModel checkpoints say ``decoder.*``, Int8OPTForCausalLM
    ones ``model.decoder.*``; either loads into either class."""
    if key in targets:
        return key
    if "model." + key in targets:
        return "model." + key
    if key.startswith("model.") and key[len("model."):] in targets:
        return key[len("model."):]
    return None


def _fit(name: str, t: torch.Tensor, want: torch.Size) -> torch.Tensor:
    if t.shape == want:
        return t
    leaf = name.rsplit(".", 1)[-1]
    # [N] <-> [1, N] biases and 0-d <-> [1] scales are the same data
    if t.numel() == want.numel() and (leaf == "bias" or want.numel() == 1):
        return t.reshape(want)
    raise ValueError(f"{name}: checkpoint holds shape {tuple(t.shape)}, the model expects {tuple(want)}")


def _rank_marker(directory: str) -> Optional[Tuple[int, int]]:
    """(size, rank) if `directory` is one rank's part written by write_rank_shards, else None."""
    path = os.path.join(directory, CONFIG_NAME)
    if not os.path.isfile(path):
        return None
    with open(path) as f:
        mark = json.load(f).get("tensor_parallel")
    return (int(mark["size"]), int(mark["rank"])) if mark else None


@torch.no_grad()
def load_into(model: torch.nn.Module, directory: str, tp: Optional[TensorParallel] = None,
              strict: bool = True) -> Tuple[List[str], List[str]]:
    """Fills `model` (already built with the same `tp`) from the checkpoint in `directory`.
    Returns (missing keys, unexpected keys); with strict=True either being non-empty raises
    (``lm_head.weight`` may always be absent: it is the token embedding)."""
    tp = tp if tp is not None else TensorParallel.single()
    presliced = _rank_marker(directory)
    if presliced is not None and presliced != (tp.size, tp.rank):
        raise ValueError(f"{directory} holds rank {presliced[1]} of {presliced[0]}; "
                         f"this process is rank {tp.rank} of {tp.size}")
    files = _Files(directory)
    targets = model.state_dict(keep_vars=True)
    seen, unexpected = set(), []
    try:
        for key in files.names:
            name = _target_name(key, targets)
            if name is None:
                if not key.endswith("lm_head.weight"):   # a causal-LM checkpoint read into the bare model
                    unexpected.append(key)
                continue
            dst = targets[name]
            src = files.source(key)
            dim = tp.shard_dim(name) if tp.size > 1 and presliced is None else None
            if dim is not None:
                d = dim % len(src.shape)
                start, stop = tp.shard_range(src.shape[d])
                t = src.read(d, start, stop)
            else:
                t = src.read()
            t = _fit(name, t, dst.shape)
            if dst.dtype.is_floating_point != t.dtype.is_floating_point or \
                    (not dst.dtype.is_floating_point and dst.dtype != t.dtype):
                raise ValueError(f"{name}: checkpoint dtype {t.dtype} does not fit the model's {dst.dtype}")
            dst.copy_(t)
            seen.add(name)
    finally:
        files.close()
    missing = [k for k in targets if k not in seen and not k.endswith("lm_head.weight")]
    if strict and (missing or unexpected):
        raise KeyError(f"{directory}: missing keys {missing[:5]}{'...' if len(missing) > 5 else ''}, "
                       f"unexpected keys {unexpected[:5]}{'...' if len(unexpected) > 5 else ''}")
    return missing, unexpected


def load_pretrained(cls, directory: str, device="cuda", torch_dtype: Optional[torch.dtype] = None,
                    tp: Optional[TensorParallel] = None, strict: bool = True, device_map=None):
    """``cls.from_pretrained``: builds `cls` (Int8OPTModel or Int8OPTForCausalLM) on `device` and loads
    the checkpoint.  `torch_dtype` is the dtype of the floating-point parameters (embeddings, final
    LayerNorm, lm_head), default: the one config.json names, else float32; the int8 / int32 / fp32
    buffers of the quantised operators keep their own dtypes, as with the reference
    (nn/linear.py:30-34).  `device_map` is accepted for call compatibility
    (benchmark/bench_opt.py:35-36): "auto" means `device`."""
    if device_map not in (None, "auto"):
        device = device_map if not isinstance(device_map, dict) else device_map.get("", device)
    config, named = read_config(directory)
    dtype = torch_dtype or named or torch.float32
    with torch.device(device):
        model = cls(config, tp=tp)
    cast_float_parameters(model, dtype)
    load_into(model, directory, tp=tp, strict=strict)
    return model.eval()


def cast_float_parameters(model: torch.nn.Module, dtype: torch.dtype):
    """Casts the nn.Parameters (embeddings, final LayerNorm, projections, lm_head) to `dtype`, keeps
    the lm_head tied, and leaves every buffer of the quantised operators alone."""
    for p in model.parameters():
        if p.dtype.is_floating_point and p.dtype != dtype:
            p.data = p.data.to(dtype)
    return model


# --------------------------------------------------------------------------- saving
def _plain(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().to("cpu")
    if not t.is_contiguous() or t.untyped_storage().nbytes() != t.numel() * t.element_size():
        t = t.contiguous().clone()   # a view into a larger (fused q/k/v) tensor: store only its own bytes
    return t


def _plan(sizes: Dict[str, int], max_shard_bytes: int) -> List[List[str]]:
    """Greedy split in state-dict order (layers stay together) into files of at most max_shard_bytes."""
    plan: List[List[str]] = [[]]
    size = 0
    for k, nbytes in sizes.items():
        if plan[-1] and size + nbytes > max_shard_bytes:
            plan.append([])
            size = 0
        plan[-1].append(k)
        size += nbytes
    return plan


def _write(directory: str, config: dict, plan: List[List[str]], fetch, total_bytes: int,
           safe_serialization: bool) -> List[str]:
    """Writes config.json and one file per entry of `plan`; fetch(name) returns the tensor to store, so
    only one file's tensors are in host memory at a time."""
    os.makedirs(directory, exist_ok=True)
    for stale in os.listdir(directory):   # a previous save with another split must not be picked up
        if re.fullmatch(r"(model|pytorch_model)(-\d{5}-of-\d{5})?\.(safetensors|bin)(\.index\.json)?", stale):
            os.remove(os.path.join(directory, stale))
    with open(os.path.join(directory, CONFIG_NAME), "w") as f:
        json.dump(config, f, indent=2, sort_keys=True)
    ext = "safetensors" if safe_serialization else "bin"
    stem = "model" if safe_serialization else "pytorch_model"

    def write(fname, names):
        tensors = {k: _plain(fetch(k)) for k in names}
        path = os.path.join(directory, fname)
        if safe_serialization:
            from safetensors.torch import save_file
            save_file(tensors, path, metadata={"format": "pt"})
        else:
            torch.save(tensors, path)

    if len(plan) == 1:
        write(f"{stem}.{ext}", plan[0])
        return [f"{stem}.{ext}"]
    weight_map, files = {}, []
    for i, names in enumerate(plan):
        fname = f"{stem}-{i + 1:05d}-of-{len(plan):05d}.{ext}"
        write(fname, names)
        files.append(fname)
        weight_map.update({k: fname for k in names})
    with open(os.path.join(directory, _ST_INDEX if safe_serialization else _BIN_INDEX), "w") as f:
        json.dump({"metadata": {"total_size": total_bytes}, "weight_map": weight_map}, f, indent=2, sort_keys=True)
    return files


def save_pretrained(model: torch.nn.Module, directory: str, max_shard_bytes: int = 5 << 30,
                    safe_serialization: bool = True) -> List[str]:
    """Writes config.json and the state dict of a single-GPU model in the transformers layout,
    split into files of at most `max_shard_bytes` (with an index) when it is larger than that.
    Returns the tensor file names."""
    tp = None
    for m in model.modules():
        tp = getattr(m, "tp", None) or tp
    if tp is not None and tp.size > 1:
        raise RuntimeError("save_pretrained writes whole models; this one holds rank "
                           f"{tp.rank} of {tp.size} of the split weights")
    state = model.state_dict()
    for k in [k for k in state if k.endswith("lm_head.weight")]:
        emb = k[:-len("lm_head.weight")] + "model.decoder.embed_tokens.weight"
        if emb in state and state[emb].data_ptr() == state[k].data_ptr():
            del state[k]      # tied: stored once, as the embedding
    floats = [t.dtype for k, t in state.items() if k.endswith("embed_tokens.weight")]
    config = config_dict(model.config, floats[0] if floats else torch.float32, type(model).__name__)
    sizes = {k: t.numel() * t.element_size() for k, t in state.items()}
    return _write(directory, config, _plan(sizes, max_shard_bytes), state.__getitem__, sum(sizes.values()),
                  safe_serialization)


def rank_directory(directory: str, size: int, rank: int) -> str:
    return os.path.join(directory, f"rank-{rank:05d}-of-{size:05d}")


def write_rank_shards(source: str, destination: str, size: int, max_shard_bytes: int = 5 << 30,
                      safe_serialization: bool = True) -> List[str]:
    """Splits the whole-model checkpoint in `source` into `size` per-rank checkpoints
    ``destination/rank-0000r-of-0000n`` (same layout; config.json additionally records
    ``"tensor_parallel": {"size": n, "rank": r}``), so that a later start-up reads plain files with no
    slicing.  ``from_pretrained(rank_directory(...), tp=...)`` loads one.  Works tensor by tensor: host
    memory holds one output file at a time."""
    with open(os.path.join(source, CONFIG_NAME)) as f:
        config = json.load(f)
    if "tensor_parallel" in config:
        raise ValueError(f"{source} is already a per-rank checkpoint")
    files = _Files(source)
    out = []
    try:
        for rank in range(size):
            tp = TensorParallel(size, rank)

            def fetch(k, tp=tp):
                src = files.source(k)
                dim = tp.shard_dim(k)
                if dim is None or len(src.shape) == 0:
                    return src.read()
                d = dim % len(src.shape)
                return src.read(d, *tp.shard_range(src.shape[d]))

            sizes = {}
            for k in files.names:
                src = files.source(k)
                n = src.itemsize
                for v in src.shape:
                    n *= v
                sizes[k] = n // size if tp.shard_dim(k) is not None else n
            target = rank_directory(destination, size, rank)
            _write(target, dict(config, tensor_parallel={"size": size, "rank": rank}),
                   _plan(sizes, max_shard_bytes), fetch, sum(sizes.values()), safe_serialization)
            out.append(target)
    finally:
        files.close()
    return out
