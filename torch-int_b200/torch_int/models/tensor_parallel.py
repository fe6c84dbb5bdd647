"""Tensor parallelism for the Int8 OPT models: one process per GPU, NCCL over
NVLink for the two reductions per layer.

Partitioning (Megatron style): q/k/v and fc1 are split by OUTPUT features
(whole attention heads per rank), out_proj and fc2 by INPUT features.  The
row-parallel GEMMs emit int32 partial sums, which are all-reduced; integer
addition is associative, so the reduced accumulator is bit-identical to the
single-GPU accumulator for every rank count and reduction order, and the fp32
epilogue (scale, bias, residual add, LayerNorm, quantise) then runs once on the
reduced value on every rank.  The reference has no multi-GPU path
(no torch.distributed call in torch_int/); this file is new functionality.
"""
from typing import Dict, Optional

import torch
import torch.distributed as dist


class TensorParallel:
    def __init__(self, size: int = 1, rank: int = 0, group=None):
        self.size = size
        self.rank = rank
        self.group = group

    @staticmethod
    def single() -> "TensorParallel":
        return TensorParallel(1, 0, None)

    @staticmethod
    def from_world(group=None) -> "TensorParallel":
        """Context spanning the default (or the given) process group."""
        if not dist.is_available() or not dist.is_initialized():
            return TensorParallel.single()
        return TensorParallel(dist.get_world_size(group), dist.get_rank(group), group)

    def all_reduce_int32(self, partial: torch.Tensor) -> torch.Tensor:
        """Sums int32 partial accumulators over the ranks, in place."""
        if self.size == 1:
            return partial
        if partial.dtype != torch.int32:
            raise RuntimeError("tensor-parallel partial sums must be int32")
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        return partial

    # ------------------------------------------------------------- weight sharding
    def _rows(self, t: torch.Tensor) -> torch.Tensor:
        n = t.shape[0]
        assert n % self.size == 0, (n, self.size)
        s = n // self.size
        return t[self.rank * s:(self.rank + 1) * s].contiguous()

    def _cols(self, t: torch.Tensor) -> torch.Tensor:
        n = t.shape[-1]
        assert n % self.size == 0, (n, self.size)
        s = n // self.size
        return t[..., self.rank * s:(self.rank + 1) * s].contiguous()

    def shard_state_dict(self, full: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """This rank's slice of a single-GPU Int8 OPT state dict.  Column-parallel
        linears (q/k/v/fc1): rows of `weight`, entries of the [1,N] `bias`.
        Row-parallel linears (out_proj/fc2): columns of `weight`; the fp32 bias is
        kept whole on every rank (it is applied after the reduction).  Everything
        else (scales, LayerNorm parameters, embeddings) is replicated."""
        if self.size == 1:
            return dict(full)
        out = {}
        for name, t in full.items():
            parts = name.split(".")
            leaf, owner = parts[-1], parts[-2] if len(parts) > 1 else ""
            if owner in ("q_proj", "k_proj", "v_proj", "fc1") and leaf == "weight":
                out[name] = self._rows(t)
            elif owner in ("q_proj", "k_proj", "v_proj", "fc1") and leaf == "bias":
                out[name] = self._cols(t.reshape(1, -1))
            elif owner in ("out_proj", "fc2") and leaf == "weight":
                out[name] = self._cols(t)
            else:
                out[name] = t
        return out
