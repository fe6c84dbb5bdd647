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
    def __init__(self, size: int = 1, rank: int = 0, group=None, max_chunks: int = 8,
                 min_pipeline_tokens: int = 1024):
        self.size = size
        self.rank = rank
        self.group = group
        self.max_chunks = max_chunks  # pipeline depth of the layer loop (groups of sequences)
        # below this many tokens per group (decode steps, short prompts) the exchanges are latency
        # bound and one all-reduce per exchange point is faster than the pipelined form
        self.min_pipeline_tokens = min_pipeline_tokens
        self._comm_streams = {}

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

    def comm_stream(self, device):
        """The stream the exchanges of the pipelined layer loop are enqueued on."""
        key = torch.device(device).index
        if key not in self._comm_streams:
            self._comm_streams[key] = torch.cuda.Stream(device=device)
        return self._comm_streams[key]

    def plan_chunks(self, batch: int, tgt_len: int) -> int:
        """Number of sequence groups for the pipelined layer loop: the largest divisor
        of `batch` up to max_chunks whose groups have a token count divisible by the
        rank count (rows are reduce-scattered evenly).  0 = use the all-reduce path."""
        for c in range(min(self.max_chunks, batch), 0, -1):
            tokens = (batch // c) * tgt_len
            if batch % c == 0 and tokens % self.size == 0 and tokens >= self.min_pipeline_tokens:
                return c
        return 0

    def reduce_scatter_int32(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum of the ranks' int32 partials [M, E]; rank r receives rows [r*M/n, (r+1)*M/n)."""
        if partial.dtype != torch.int32 or partial.shape[0] % self.size != 0:
            raise RuntimeError("reduce_scatter_int32 needs an int32 tensor whose rows divide evenly over the ranks")
        out = torch.empty((partial.shape[0] // self.size,) + tuple(partial.shape[1:]), dtype=torch.int32,
                          device=partial.device)
        dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def all_gather_into(self, full: torch.Tensor, shard: torch.Tensor) -> torch.Tensor:
        """Concatenates the ranks' row shards into `full` (rank order)."""
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

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
