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
import contextlib
import json
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist


class StreamTrace:
    """Timeline of the pipelined layer loop: named spans bracketed by CUDA events on the stream they
    run on (an event costs no synchronisation and no launch).  dump() resolves the events after a
    device synchronise and writes Chrome trace-event JSON (chrome://tracing, Perfetto), one row per
    stream, so exposed exchange time and idle gaps of the compute stream can be read off directly.
    `new_event` is injectable so that the bookkeeping can be tested without a GPU."""

    def __init__(self, new_event=None):
        self._new_event = new_event or (lambda: torch.cuda.Event(enable_timing=True))
        self.spans = []       # (name, row, args, start event, end event)
        self.origin = None    # (stream, event) recorded by the first span

    @contextlib.contextmanager
    def span(self, name: str, row: str, stream, **args):
        start, end = self._new_event(), self._new_event()
        start.record(stream)
        if self.origin is None:
            self.origin = start
        try:
            yield
        finally:
            end.record(stream)
            self.spans.append((name, row, args, start, end))

    def events(self, pid: int = 0):
        """Chrome trace events (microseconds from the first span's start).  Call after a synchronise."""
        rows = {}
        out = []
        for name, row, args, start, end in self.spans:
            tid = rows.setdefault(row, len(rows))
            ts = self.origin.elapsed_time(start) * 1e3
            out.append({"name": name, "ph": "X", "pid": pid, "tid": tid, "ts": ts,
                        "dur": max(0.0, start.elapsed_time(end) * 1e3), "args": args})
        for row, tid in rows.items():
            out.append({"name": "thread_name", "ph": "M", "pid": pid, "tid": tid, "args": {"name": row}})
        return out

    def summary(self):
        """Per row: busy microseconds (sum of span durations) and the extent from first start to last end."""
        acc = {}
        for e in self.events():
            if e["ph"] != "X":
                continue
            r = acc.setdefault(e["tid"], {"busy_us": 0.0, "first_us": e["ts"], "last_us": e["ts"] + e["dur"],
                                          "by_name": {}})
            r["busy_us"] += e["dur"]
            r["first_us"] = min(r["first_us"], e["ts"])
            r["last_us"] = max(r["last_us"], e["ts"] + e["dur"])
            r["by_name"][e["name"]] = r["by_name"].get(e["name"], 0.0) + e["dur"]
        names = {e["tid"]: e["args"]["name"] for e in self.events() if e["ph"] == "M"}
        return {names[t]: v for t, v in acc.items()}

    def dump(self, path: str, pid: int = 0):
        with open(path, "w") as f:
            json.dump({"traceEvents": self.events(pid), "summary": self.summary()}, f)


_NO_SPAN = contextlib.nullcontext()


class TensorParallel:
    def __init__(self, size: int = 1, rank: int = 0, group=None, max_chunks: int = 4,
                 min_pipeline_tokens: int = 1024):
        self.size = size
        self.rank = rank
        self.group = group
        # pipeline depth of the layer loop (groups of sequences); TI_TP_CHUNKS overrides
        self.max_chunks = int(os.environ.get("TI_TP_CHUNKS", max_chunks))
        # below this many tokens per group (decode steps, short prompts) the exchanges are latency
        # bound and one all-reduce per exchange point is faster than the pipelined form
        self.min_pipeline_tokens = min_pipeline_tokens
        self._comm_streams = {}
        self._workspaces = {}
        # fuse the exchanges into the GEMM epilogue / LayerNorm kernel through peer stores
        self.use_peer_memory = os.environ.get("TI_TP_PEER_MEMORY", "1") != "0"
        # how the partial sums reach their owner: "copy" = local GEMM output, then contiguous peer
        # copies on the communication stream (copy engines; overlaps all compute of the other groups);
        # "epilogue" = the GEMM epilogue stores straight into the owners' memory
        self.peer_mode = os.environ.get("TI_TP_PEER_MODE", "copy")
        # SMs the GEMM grids may use while exchanges overlap them (0 = all); TI_TP_GEMM_SMS overrides
        self.gemm_sm_limit = int(os.environ.get("TI_TP_GEMM_SMS", "0"))
        # 1: one communication stream carries copy -> barrier -> reduce+LayerNorm -> barrier of each
        # exchange back to back.  2 (default): the copies (+ first barrier) and the reduce kernel (+ second
        # barrier) run on two streams, so the copies of the next group overlap the reduction of this one
        # (8 ranks, OPT-175B: one stream is busy 440 ms of a 455 ms step; two streams give 445 ms).
        self.comm_streams = int(os.environ.get("TI_TP_COMM_STREAMS", "2"))
        # False (default): barrier kernel -> reduce kernel -> barrier kernel.  True: the two barriers of
        # an exchange are folded into the reduce kernel (one launch per exchange after the copies).
        # Measured at 8 ranks (OPT-175B, batch 16 x 1024): 455 ms per step with the separate barrier
        # kernels, 470 ms folded - while a folded kernel waits for a slower rank, its 512 CTAs hold
        # the registers the next GEMM needs, whereas a waiting barrier kernel is one warp.
        self.fused_sync = os.environ.get("TI_TP_FUSED_SYNC", "0") == "1"
        # replay tensor-parallel decode steps (which contain NCCL all-reduces) from a CUDA graph: eager
        # steps are bound by the host's launch rate (31 ms per step at 4 and 8 ranks of OPT-175B)
        self.decode_graph = os.environ.get("TI_TP_DECODE_GRAPH", "1") != "0"
        # a StreamTrace while a forward pass is being traced, else None
        self.trace: Optional[StreamTrace] = None
        # language-model head split by vocabulary rows: each rank multiplies with its 1/size of the
        # (tied, replicated) embedding table and the logits are all-gathered.  The floating-point GEMM
        # of a shard may round differently from the whole one, so logits are then equal to the
        # single-GPU ones only to fp32 / fp16 accuracy, not bit for bit: opt-in (TI_TP_VOCAB_PARALLEL=1).
        self.vocab_parallel = os.environ.get("TI_TP_VOCAB_PARALLEL", "0") == "1"

    def span(self, name: str, row: str, stream, **args):
        """Context manager: a span of the timeline when tracing is on, otherwise nothing."""
        return self.trace.span(name, row, stream, **args) if self.trace is not None else _NO_SPAN

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

    def comm_stream(self, device, index: int = 0):
        """The stream(s) the exchanges of the pipelined layer loop are enqueued on."""
        key = (torch.device(device).index, index)
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
        rows = partial.shape[0] // self.size
        if dist.get_backend(self.group) == "gloo":
            # CPU ranks (the host-logic tests): gloo has no reduce-scatter; integer sums are exact either way
            total = partial.clone()
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group)
            return total[self.rank * rows:(self.rank + 1) * rows].contiguous()
        out = torch.empty((rows,) + tuple(partial.shape[1:]), dtype=torch.int32, device=partial.device)
        dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def all_gather_into(self, full: torch.Tensor, shard: torch.Tensor) -> torch.Tensor:
        """Concatenates the ranks' row shards into `full` (rank order)."""
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

    def vocab_parallel_logits(self, hidden: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """hidden [..., E] x table[V, E]^T -> logits [..., V], each rank computing the columns of its
        V/size rows of `table` (a view: the table stays whole and tied to the embedding) followed by an
        all-gather.  Falls back to the whole product when V does not divide over the ranks."""
        v = table.shape[0]
        if self.size == 1 or v % self.size != 0:
            return torch.nn.functional.linear(hidden, table)
        v0, v1 = self.shard_range(v)
        lead = hidden.shape[:-1]
        local = torch.nn.functional.linear(hidden.reshape(-1, hidden.shape[-1]), table[v0:v1])   # [tokens, V/size]
        tokens = local.shape[0]
        gathered = torch.empty((self.size * tokens, v1 - v0), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(gathered, local.contiguous(), group=self.group)   # rank blocks along dim 0
        # [size, tokens, V/size] -> [tokens, size * V/size]
        return gathered.view(self.size, tokens, v1 - v0).permute(1, 0, 2).reshape(*lead, v)

    def agree_max(self, value: int, device) -> int:
        """Maximum of a small integer over the ranks (one collective): the way every rank reaches the
        same decision from per-rank observations."""
        if self.size == 1:
            return int(value)
        t = torch.tensor([int(value)], dtype=torch.int32, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return int(t.item())

    def peer_workspace(self, chunks: int, mc: int, e: int, device):
        """Peer-accessible buffers for the fused exchange of the pipelined layer loop, or
        None when symmetric memory is unavailable (then NCCL collectives are used).

        Every rank must call this at the same point: whether the peer-memory path is used is decided
        COLLECTIVELY.  A rank whose allocation or set-up failed reports that through a reduction over
        the ranks, and then all ranks fall back together; a rank never switches paths on its own (its
        peers would wait for it in a barrier while it waits for them in a collective)."""
        if not self.use_peer_memory:
            return None
        key = (chunks, mc, e, torch.device(device).index)
        ws = self._workspaces.get(key)
        if ws is None:
            ws = PeerWorkspace.create(self, chunks, mc, e, device)
            if ws is None:
                import warnings
                warnings.warn("tensor parallel: peer memory unavailable on at least one rank; "
                              "all ranks use NCCL collectives")
                self.use_peer_memory = False
                return None
            self._workspaces[key] = ws
        return ws

    def check_exchange(self, ws, device):
        """Reads the kernels' status word, agreed over the ranks, after a forward pass that used the
        peer-memory exchange `ws`.  Non-zero (a bounded wait of a barrier ran out on some rank: the
        activations of that pass are not trustworthy) switches ALL ranks to the NCCL exchange and raises.
        Called for the first pass of every workspace, and for every pass when TI_TP_CHECK_EVERY_PASS=1."""
        from .. import _CUDA as C
        status = self.agree_max(C.device_status(reset=True), device)
        ws.checked = True
        if status != 0:
            self.use_peer_memory = False
            self._workspaces.clear()
            raise RuntimeError(f"tensor parallel: the peer-memory exchange reported status {status} (a bounded wait "
                               "ran out); the results of this pass are invalid.  All ranks now use NCCL collectives: "
                               "repeat the call.")

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

    @staticmethod
    def shard_dim(name: str):
        """Which dimension of the Int8 OPT buffer `name` is split over the ranks (None = replicated).
        Column-parallel linears (q/k/v/fc1): rows of `weight` (0) and entries of `bias` (-1).
        Row-parallel linears (out_proj/fc2): columns of `weight` (1); their fp32 bias is kept whole
        on every rank, since it is applied after the reduction.  Scales, LayerNorm parameters and
        embeddings are replicated."""
        parts = name.split(".")
        leaf, owner = parts[-1], parts[-2] if len(parts) > 1 else ""
        if owner in ("q_proj", "k_proj", "v_proj", "fc1"):
            return 0 if leaf == "weight" else -1 if leaf == "bias" else None
        if owner in ("out_proj", "fc2") and leaf == "weight":
            return 1
        return None

    def shard_range(self, n: int):
        """[start, stop) of this rank's part of an extent-n split dimension."""
        if n % self.size != 0:
            raise ValueError(f"extent {n} cannot be split over {self.size} ranks")
        s = n // self.size
        return self.rank * s, (self.rank + 1) * s

    def shard_state_dict(self, full: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """This rank's slice (see shard_dim) of a single-GPU Int8 OPT state dict."""
        if self.size == 1:
            return dict(full)
        out = {}
        for name, t in full.items():
            dim = self.shard_dim(name)
            if dim == 0:
                out[name] = self._rows(t)
            elif dim == -1:
                out[name] = self._cols(t.reshape(1, -1))
            elif dim == 1:
                out[name] = self._cols(t)
            else:
                out[name] = t
        return out


class PeerWorkspace:
    """Symmetric (same layout on every rank, mapped into every rank) buffers of the fused
    tensor-parallel exchange:
      stage [chunks][n][ms][e] int32  slab s of chunk c receives rank s's partial sums of my rows
      h8    [chunks][mc][e]   int8   the LayerNorm-quantise output of all rows (every owner writes its rows)
      pads  [n] uint32               barrier words
    Allocated with torch's symmetric memory (cuMem mappings exchanged between the processes);
    all traffic is plain peer loads/stores issued by this library's kernels."""

    @classmethod
    def create(cls, tp: "TensorParallel", chunks: int, mc: int, e: int, device):
        """Collective constructor: returns the workspace on every rank, or None on every rank.  Each
        phase that can fail on one rank alone (allocation, mapping, the barrier preflight) ends with a
        reduction of a failure flag over the ranks, so that no rank is left waiting for one that gave up."""
        ws = object.__new__(cls)
        ws.checked = False
        dev = torch.device(device)
        err = None
        try:
            ws._allocate(tp, chunks, mc, e, dev)
        except Exception as exc:  # noqa: BLE001 - any local failure means "all ranks fall back"
            err = exc
        if tp.agree_max(0 if err is None else 1, dev) != 0:
            return None
        try:
            ws._map_and_preflight()
        except Exception as exc:  # noqa: BLE001
            err = exc
        if tp.agree_max(0 if err is None else 1, dev) != 0:
            return None
        return ws

    def _allocate(self, tp, chunks, mc, e, device):
        import torch.distributed._symmetric_memory as symm
        from .. import _CUDA as C
        self._C = C
        n = tp.size
        ms = mc // n
        self.tp, self.chunks, self.mc, self.ms, self.e, self.device = tp, chunks, mc, ms, e, device
        stage_bytes = chunks * n * ms * e * 4
        h8_bytes = chunks * mc * e
        self.stage_bytes, self.h8_bytes = stage_bytes, h8_bytes
        self.stage_off = 0
        self.h8_off = (stage_bytes + 255) // 256 * 256
        self.pad_off = (self.h8_off + h8_bytes + 255) // 256 * 256
        total = self.pad_off + 256
        self.group = tp.group if tp.group is not None else dist.group.WORLD
        self.buf = symm.empty(total, dtype=torch.uint8, device=self.device)

    def _map_and_preflight(self):
        import torch.distributed._symmetric_memory as symm
        C, tp, group = self._C, self.tp, self.group
        chunks, n, ms, e, mc = self.chunks, tp.size, self.ms, self.e, self.mc
        self.handle = symm.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.stage = self.buf[:self.stage_bytes].view(torch.int32).view(chunks, n, ms, e)
        self.h8 = self.buf[self.h8_off:self.h8_off + self.h8_bytes].view(torch.int8).view(chunks, mc, e)
        self.buf[self.pad_off:].zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)  # every rank's pads are zero before the first barrier kernel
        # four independent barrier channels of 64 bytes (up to 16 ranks) each, with their own epochs:
        # barriers issued on different streams must not share words
        self.epochs = [0] * 4
        self.channel_pads = [[p + self.pad_off + 64 * ch for p in self.ptrs] for ch in range(4)]
        self.pad_ptrs = self.channel_pads[0]
        # CTA counters of the reduce kernel with folded-in synchronisation (one per channel)
        self.counters = torch.zeros(4, dtype=torch.int32, device=self.device)
        # Preflight: a few barriers over the fresh pads, with a generous time limit (the first kernels
        # of a process load lazily, so the ranks may reach them seconds apart).  If peer stores or
        # loads do not work on this machine the (bounded) waits give up and set the status word; every
        # rank then learns of it through the reduction in create().
        for _ in range(3):
            self.barrier(limit_ms=self.FIRST_LIMIT_MS)
        status = C.device_status(reset=True)
        if status != 0:
            raise RuntimeError(f"peer-memory barrier preflight failed (status {status})")
        # every rank's stage as a tensor of this process (peer mappings), for contiguous peer copies
        self.peer_stage = [self.handle.get_buffer(o, (chunks, n, ms, e), torch.int32, 0) for o in range(n)]

    # time limits of a barrier's wait: the first barriers of a workspace tolerate start-up skew
    # between the ranks; TI_TP_BARRIER_LIMIT_MS sets the limit of all later ones
    FIRST_LIMIT_MS = 20000
    LIMIT_MS = int(os.environ.get("TI_TP_BARRIER_LIMIT_MS", "2000"))

    def scatter_ptrs(self, c):
        """Where the GEMM epilogue writes row block o of chunk c: slab [my rank] of owner o's stage."""
        n, ms, e, r = self.tp.size, self.ms, self.e, self.tp.rank
        return [p + self.stage_off + ((c * n + r) * ms * e) * 4 for p in self.ptrs]

    def q_dst_ptrs(self, c):
        return [p + self.h8_off + c * self.mc * self.e for p in self.ptrs]

    def push_partials(self, c, acc):
        """Copies row block o of the local partial sums acc [mc, e] into slab [my rank] of owner o's
        stage, for every o (contiguous device-to-device copies on the current stream)."""
        r, ms = self.tp.rank, self.ms
        for i in range(self.tp.size):
            o = (r + 1 + i) % self.tp.size  # start with the right-hand neighbour: spreads the link load
            self.peer_stage[o][c, r].copy_(acc[o * ms:(o + 1) * ms], non_blocking=True)

    def exchange_reduce(self, c, scale, bias, residual, ln, channel: int = 2):
        """The second half of an exchange as ONE kernel on the current stream (after the copies of
        push_partials in stream order): announce, wait for all ranks, reduce + LayerNorm-quantise chunk
        c's rows of this rank into every rank's activation buffer, wait until all ranks are complete.
        Returns the new residual rows.  All calls of one channel come from one stream, in the same order
        on every rank."""
        self.epochs[channel] += 1
        limit_ms = self.LIMIT_MS if self.checked else self.FIRST_LIMIT_MS
        return self._C.tp_exchange_reduce_layernorm_q(
            self.stage[c], self.tp.size, self.ms * self.e, scale, bias, residual, ln.weight, ln.bias, ln.eps,
            self.q_dst_ptrs(c), self.tp.rank * self.ms, self.channel_pads[channel], self.tp.rank,
            self.epochs[channel], self.counters[channel:channel + 1], limit_ms=limit_ms)

    def barrier(self, channel: int = 0, limit_ms: Optional[int] = None):
        """Enqueues a bounded barrier over all ranks on the current stream.  All barriers of one
        channel must be issued from one stream, in the same order on every rank.  Until the first
        forward pass over this workspace has been checked, the generous start-up limit applies."""
        self.epochs[channel] += 1
        if limit_ms is None:
            limit_ms = self.LIMIT_MS if self.checked else self.FIRST_LIMIT_MS
        self._C.tp_barrier(self.channel_pads[channel], self.tp.rank, self.epochs[channel], self.device,
                           limit_ms=limit_ms)
