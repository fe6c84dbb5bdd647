"""Benchmark of the W8A8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Workloads:
  gemm     the headline W8A8 GEMM, 4096 x 12288 x 12288, int8 output
           (linear_a8_w8_b8_o8); N GPUs run N independent replicas.
  opt30b   Int8OPTForCausalLM at the OPT-30B architecture, batch 8, 512-token
           prefill, one GPU.
  opt175b  the OPT-175B architecture, batch 16, 1024-token prefill, tensor
           parallel over N = 2/4/8 GPUs with two int32 all-reduces per layer.
The default is opt30b at N=1 and opt175b at N>1 once the model path is
available in this checkout, else gemm.

`--impl reference` times the reference semantics on the host CPU (the oracle's
C restatement, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "torch-int_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

HG = (4096, 12288, 12288)  # M, N, K of the headline GEMM


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


_T0 = time.time()
_RANK = int(os.environ.get("RANK", "0"))


def progress(msg):
    """One line on stderr per phase (rank and seconds since start): a run that stops early shows where."""
    sys.stderr.write(f"[bench rank {_RANK} +{time.time() - _T0:6.1f}s] {msg}\n")
    sys.stderr.flush()


class Watchdog:
    """Ends the process if a phase has not finished in time (a hung collective or a machine problem must
    not hold the GPUs until an outer limit kills the job).  Once the prefill measurement exists, rank 0
    prints that line - with the unfinished leg reported as an error inside it - and every rank exits 0,
    so a late failure does not lose the measurement."""

    def __init__(self, rank):
        self.rank = rank
        self.line = None          # the JSON line as far as it is known (rank 0)
        self.salvageable = False  # True once the prefill + end-to-end legs are measured (all ranks)
        self.phase = "start"
        self.timer = None
        self.lock = threading.Lock()

    def arm(self, seconds, phase):
        with self.lock:
            if self.timer is not None:
                self.timer.cancel()
            self.phase = phase
            self.timer = threading.Timer(seconds, self._fire, args=(seconds, phase))
            self.timer.daemon = True
            self.timer.start()

    def disarm(self):
        with self.lock:
            if self.timer is not None:
                self.timer.cancel()
                self.timer = None

    def _fire(self, seconds, phase):
        msg = f"bench.py watchdog: phase '{phase}' not finished after {seconds} s, giving up"
        sys.stderr.write(msg + "\n")
        sys.stderr.flush()
        if self.salvageable:
            if self.rank == 0 and self.line is not None:
                self.line.setdefault("legs_failed", {})[phase] = msg
                print(json.dumps(self.line), flush=True)
            os._exit(0)
        if self.rank == 0:
            print(json.dumps({"error": msg}), flush=True)
        os._exit(3)


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


# DRAM traffic per launch of gemm_i8_kernel, from ncu (dram__bytes_read.sum + dram__bytes_write.sum of one
# captured launch; the summaries under profiles/ give the commands).  Keyed by (M, N, K).
NCU_GEMM_TRAFFIC_BYTES = {
    (4096, 12288, 12288): 462.1e6,   # profiles/gemm_i8_pair_4096x12288x12288.md
    (4096, 28672, 7168): 344.0e6,    # profiles/gemm_i8_pair_fc1_4096x28672x7168.md
}


def gemm_traffic_bytes(m, n, k):
    return NCU_GEMM_TRAFFIC_BYTES.get((m, n, k))


def headline_gemm_sustained(device, peaks, launches=600):
    """The headline W8A8 GEMM (4096 x 12288 x 12288, int8 out) back to back for `launches` launches with the
    SM clock sampled meanwhile: the sustained TOP/s under the power cap."""
    from torch_int import _CUDA as C
    m, n, k = HG
    gd = torch.Generator(device=device).manual_seed(11)
    x = torch.randint(-127, 128, (m, k), generator=gd, dtype=torch.int8, device=device)
    w = torch.randint(-127, 128, (n, k), generator=gd, dtype=torch.int8, device=device)
    b = torch.randint(-127, 128, (n,), generator=gd, dtype=torch.int8, device=device)
    for _ in range(5):
        C.linear_a8_w8_b8_o8(x, w, b, 1e-4, 0.01)
    torch.cuda.synchronize()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        C.linear_a8_w8_b8_o8(x, w, b, 1e-4, 0.01)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / launches
    tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    sustained = 2.0 * peaks["bf16_tflops_sustained"]
    return {"shape": [m, n, k], "launches": launches, "ms": round(ms, 4), "tops": round(tops, 1),
            "frac_of_sustained_peak": round(tops / sustained, 4), "sustained_peak": round(sustained, 1),
            "frac_of_nominal_4500": round(tops / 4500.0, 4), "sm_mhz_median": clocks.get("sm_mhz"),
            "reasons": clocks.get("reasons"), "traffic": gemm_traffic_bytes(m, n, k),
            "algorithmic_bytes": float(m * k + n * k + n + m * n)}


# ----------------------------------------------------------------------------- GEMM workload
class GemmWorkload:
    name = "w8a8_gemm_4096x12288x12288_int8out"
    metric = "w8a8_gemm_tops"
    unit = "TOP/s"
    dtype = "int8"
    arithmetic = "int8 x int8 -> int32 on tcgen05 (kind::i8), fp32 epilogue, int8 out"
    scaling = "weak"

    def __init__(self, device):
        from torch_int import _CUDA as C
        self.C = C
        m, n, k = HG
        g = torch.Generator().manual_seed(0)
        self.x_host = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).pin_memory()
        self.y_host = torch.empty((m, n), dtype=torch.int8).pin_memory()
        gd = torch.Generator(device=device).manual_seed(1)
        self.x = self.x_host.to(device)
        self.w = torch.randint(-127, 128, (n, k), generator=gd, dtype=torch.int8, device=device)
        self.b = torch.randint(-127, 128, (n,), generator=gd, dtype=torch.int8, device=device)
        self.alpha, self.beta = 1e-4, 0.01
        self.ops_per_step = 2.0 * m * n * k
        self.h2d = self.x_host.numel()
        self.d2h = self.y_host.numel()
        self.launches_per_step = 1

    def step(self):
        return self.C.linear_a8_w8_b8_o8(self.x, self.w, self.b, self.alpha, self.beta)

    def step_e2e(self):
        x = self.x_host.to(self.x.device, non_blocking=True)
        y = self.C.linear_a8_w8_b8_o8(x, self.w, self.b, self.alpha, self.beta)
        self.y_host.copy_(y, non_blocking=True)

    def units(self, n_gpus):
        return self.ops_per_step * n_gpus / 1e12  # tera-ops per step over all replicas

    def config(self, n_gpus):
        return {"workload": self.name, "M": HG[0], "N": HG[1], "K": HG[2], "alpha": self.alpha,
                "beta": self.beta, "replicas": n_gpus, "arithmetic": self.arithmetic,
                "l2": "inputs (201 MB of int8 operands) exceed the 126 MB L2"}

    def roofline(self, ms, peaks):
        peak = 2.0 * peaks["bf16_tflops"]
        achieved = self.ops_per_step / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": "TOP/s",
                "frac": round(achieved / peak, 4), "traffic": gemm_traffic_bytes(*HG),
                "algorithmic_bytes": float(HG[0] * HG[2] + HG[1] * HG[2] + HG[1] + HG[0] * HG[1]),
                "peak_source": f"2 x cuBLAS bf16 burst of MEASURED_PEAKS.json ({peaks['source']}): "
                               "kind::i8 issues at twice the kind::f16 rate",
                "kernel": "gemm_i8_kernel<256, EPI_S8_BIAS_S8, PAIR=true> (256x256 tiles on CTA pairs)",
                "frac_of_nominal_4500": round(achieved / 4500.0, 4)}

    def cpu_sample(self):
        """Bounded sample for the CPU arm: the first `rows` rows of the same GEMM."""
        from oracle import w8a8 as O
        rows = 128
        x = self.x_host[:rows].clone()
        w, b = self.w.cpu(), self.b.cpu()
        ops = 2.0 * rows * HG[1] * HG[2]

        def run():
            return O.linear_a8_w8_b8_o8(x, w, b, self.alpha, self.beta)
        return run, ops / 1e12, f"first {rows} of {HG[0]} rows of the headline GEMM (all of W)", O.num_threads()


# ------------------------------------------------------------------------ Int8 OPT workloads
OPT_WORKLOADS = {
    # name: (architecture, batch, prefill length, decode steps)
    "opt30b": ("opt-30b", 8, 512, 128),
    "opt175b": ("opt-175b", 16, 1024, 128),
    "opt13b": ("opt-13b", 4, 512, 128),
    "opt1.3b": ("opt-1.3b", 8, 512, 32),
}
# hidden, layers, heads, ffn of the published OPT architectures (vocabulary 50272)
OPT_DIMS = {"opt-1.3b": (2048, 24, 32, 8192), "opt-13b": (5120, 40, 40, 20480),
            "opt-30b": (7168, 48, 56, 28672), "opt-175b": (12288, 96, 96, 49152)}
OPT_VOCAB = 50272


def opt_workload_name(arch, batch, seq, world):
    return f"int8_{arch}_prefill_b{batch}_s{seq}" + (f"_tp{world}" if world > 1 else "")


def opt_config_dict(key, world):
    """`config` of an OPT workload: the same dictionary for this repository's arm and for the CPU arm
    (it names the workload, not the implementation)."""
    arch, batch, seq, _ = OPT_WORKLOADS[key]
    hidden, layers, heads, ffn = OPT_DIMS[arch]
    return {"workload": opt_workload_name(arch, batch, seq, world), "architecture": arch, "layers": layers,
            "hidden": hidden, "heads": heads, "ffn": ffn, "vocab": OPT_VOCAB, "batch": batch, "prefill_len": seq,
            "arithmetic": "int8 x int8 -> int32 GEMM/BMM, fp32 epilogues and residual stream, fp16 embeddings and lm_head",
            "parallelism": f"tp{world}" if world > 1 else "single GPU",
            "weights": "random int8 uniform on [-127,127], analytic per-tensor scales x U(0.7,1.3)",
            "logits": "all positions (fp16 lm_head)",
            "l2": "per step the layers stream their int8 weights (>> 126 MB L2)"}


class OptWorkload:
    metric = "int8_opt_prefill_tokens_per_s"
    unit = "tokens/s"
    dtype = "int8"
    arithmetic = "int8 x int8 -> int32 GEMM/BMM, fp32 epilogues and residual stream, fp16 embeddings and lm_head"
    scaling = "strong"

    def __init__(self, device, key, world, rank):
        from torch_int import _CUDA as C
        from torch_int.models.random_init import opt_config, random_int8_opt
        from torch_int.models.tensor_parallel import TensorParallel
        self.C = C
        self.key = key
        arch, self.batch, self.seq, self.decode_steps = OPT_WORKLOADS[key]
        self.arch = arch
        self.cfg = opt_config(arch)
        self.world = world
        self.name = opt_workload_name(arch, self.batch, self.seq, world)
        tp = TensorParallel.from_world() if world > 1 else TensorParallel.single()
        self.tp = tp
        # ONE model over all ranks: the same seed everywhere, so that the replicated parameters (scales,
        # LayerNorm, fp32 biases, embeddings) agree; only the sharded int8 weights are drawn per rank
        self.model = random_int8_opt(self.cfg, seed=1234, device=device, tp=tp, param_dtype=torch.float16,
                                     consistent=False)
        g = torch.Generator().manual_seed(0)
        self.ids_host = torch.randint(0, self.cfg.vocab_size, (self.batch, self.seq), generator=g).pin_memory()
        self.next_host = torch.empty((self.batch,), dtype=torch.long).pin_memory()
        self.ids = self.ids_host.to(device)
        self.device = device
        self.h2d = self.ids_host.numel() * 8
        self.d2h = self.next_host.numel() * 8
        c0 = C.launch_count
        self.step()
        self.launches_per_step = C.launch_count - c0
        e, f, l = self.cfg.hidden_size, self.cfg.ffn_dim, self.cfg.num_hidden_layers
        t = self.batch * self.seq
        h, d = self.cfg.num_attention_heads, e // self.cfg.num_attention_heads
        self.gemm_ops = l * 2.0 * t * (4.0 * e * e + 2.0 * e * f)
        self.bmm_ops = l * 2.0 * 2.0 * self.batch * h * self.seq * self.seq * d
        self.head_flops = 2.0 * t * e * self.cfg.vocab_size

    def step(self):
        return self.model(self.ids).logits

    def step_e2e(self):
        ids = self.ids_host.to(self.device, non_blocking=True)
        logits = self.model(ids).logits
        self.next_host.copy_(logits[:, -1, :].argmax(dim=-1), non_blocking=True)

    def units(self, n_gpus):
        return float(self.batch * self.seq)  # tokens per step over the whole job

    def config(self, n_gpus):
        return opt_config_dict(self.key, n_gpus)

    def exchange(self):
        """How the two per-layer exchanges of the tensor-parallel run were carried out."""
        if self.world == 1:
            return "none"
        if self.tp.use_peer_memory and self.tp._workspaces:
            tail = ("one kernel: announce, wait for all ranks, reduce + LayerNorm-quantise with peer stores, wait for all ranks"
                    if self.tp.fused_sync else "barrier -> reduce+LayerNorm kernel with peer stores -> barrier")
            return (f"peer memory ({self.tp.peer_mode}): partial sums to the owners' slabs -> {tail}; "
                    f"{self.tp.comm_streams} communication stream(s), {self.tp.max_chunks} sequence groups")
        return "NCCL reduce-scatter / all-gather on a communication stream"

    def ranks_agree(self):
        """True when every rank's greedy next tokens of the last end-to-end step are the same (they must
        be: all ranks hold one model and finish with the same logits)."""
        import torch.distributed as dist
        mine = self.next_host.to(self.device)
        allv = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(allv, mine)
        return all(bool(torch.equal(allv[0], v)) for v in allv)

    def roofline(self, ms, peaks):
        """The dominant kernel is the W8A8 GEMM: the layer's largest one (fc1) is timed alone, live, in a
        burst of back-to-back launches, so the denominator is the burst figure (2 x cuBLAS bf16 burst);
        the whole step is held against the sustained figure beside it."""
        e = self.cfg.hidden_size
        t = self.batch * self.seq
        layer = self.model.model.decoder.layers[0]
        x = torch.randint(-127, 128, (t, e), dtype=torch.int8, device=self.device)
        gms = _event_time(lambda: layer.fc1._op(x), 20)
        n = layer.local_ffn
        ops = 2.0 * t * n * e
        achieved = ops / (gms * 1e-3) / 1e12
        peak = 2.0 * peaks["bf16_tflops"]
        sustained = 2.0 * peaks["bf16_tflops_sustained"]
        step_ops = (self.gemm_ops + self.bmm_ops) / self.world
        algorithmic = float(t * e + n * e + n + t * n)
        out = {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": "TOP/s",
               "frac": round(achieved / peak, 4),
               "traffic": gemm_traffic_bytes(t, n, e), "algorithmic_bytes": algorithmic,
               "kernel": f"gemm_i8_kernel (fc1: {t} x {n} x {e}, ReLU int8 epilogue)",
               "kernel_ms": round(gms, 4),
               "peak_source": f"2 x cuBLAS bf16 burst of MEASURED_PEAKS.json ({peaks['source']}): the kernel is timed "
                              "alone in a 20-launch burst; kind::i8 issues at twice the kind::f16 rate",
               "step_int8_tops_per_gpu": round(step_ops / (ms * 1e-3) / 1e12, 1),
               "step_frac_of_sustained_peak": round(step_ops / (ms * 1e-3) / 1e12 / sustained, 4),
               "sustained_peak": round(sustained, 1)}
        if self.world == 1:
            out["headline_gemm"] = headline_gemm_sustained(self.device, peaks)
        return out

    def decode_rate(self, steps=None):
        """Greedy decoding with the static int8 cache after the prefill: tokens/s over `steps` one-token
        steps (one CUDA-graph replay per step on a single GPU; eager launches under tensor parallelism)."""
        steps = steps or self.decode_steps
        model = self.model
        cache = model.new_cache(self.batch, self.seq + steps + 8)
        out = model(self.ids, past_key_values=cache, use_cache=True, last_token_only=True)
        nxt = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)
        for _ in range(3):
            nxt = model.decode_step(nxt, cache).argmax(dim=-1, keepdim=True)
        graph = None
        if self.world == 1 or self.tp.decode_graph:
            static_tok = nxt.clone()
            length = cache.length
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_next = model.decode_step(static_tok, cache).argmax(dim=-1, keepdim=True)
            cache.length = length
        torch.cuda.synchronize()
        c0 = self.C.launch_count
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps - 3):
            if graph is not None:
                static_tok.copy_(nxt)
                graph.replay()
                nxt = static_next.clone()
            else:
                nxt = model.decode_step(nxt, cache).argmax(dim=-1, keepdim=True)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (steps - 3)
        wbytes = sum(b.numel() for n, b in model.named_buffers() if b.dtype == torch.int8)
        # everything a step has to read from HBM: the int8 weights, the fp16 lm_head table (this rank's rows
        # when the head is vocabulary-parallel) and the cached keys and values at the mean length of the timed steps
        attn = model.model.decoder.layers[0].self_attn
        head = model.lm_head.weight
        head_rows = head.shape[0] // self.world if (self.world > 1 and self.tp.vocab_parallel) else head.shape[0]
        mean_len = self.seq + 3 + (steps - 2) / 2.0  # positions a timed step attends to, first to last
        kv_bytes = 2 * self.batch * attn.local_heads * attn.head_dim * mean_len * len(model.model.decoder.layers)
        hbm_bytes = wbytes + head_rows * head.shape[1] * head.element_size() + kv_bytes
        return {"decode_tokens_per_s": round(self.batch / (ms * 1e-3), 1), "decode_ms_per_step": round(ms, 3),
                "decode_steps_timed": steps - 3, "decode_weight_gb_per_s_per_gpu": round(wbytes / (ms * 1e-3) / 1e9, 1),
                "decode_hbm_gb_per_s_per_gpu": round(hbm_bytes / (ms * 1e-3) / 1e9, 1),
                "decode_mode": "CUDA graph replay" if graph is not None else "eager launches"}

    def cpu_sample(self):
        return opt_cpu_sample(self.arch, self.batch, self.seq)


def reference_layer_state(arch, seed=5):
    """State dict (the reference's buffer names) of ONE random Int8 OPT decoder layer at the dimensions
    of `arch`, built with torch alone: the CPU arm must not load this repository's package or library.
    Weights uniform int8; scales chosen so that int8 activations keep a standard deviation of a few tens."""
    import math
    h, _, heads, ffn = OPT_DIMS[arch]
    g = torch.Generator().manual_seed(seed)
    sw, sa = 127.0 / math.sqrt(3.0), 30.0
    pre = "model.decoder.layers.0"
    sd = {}

    def s8(*shape):
        return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)

    for name in ("q_proj", "k_proj", "v_proj"):
        sd[f"{pre}.self_attn.{name}.weight"] = s8(h, h)
        sd[f"{pre}.self_attn.{name}.bias"] = s8(1, h)
        sd[f"{pre}.self_attn.{name}.a"] = torch.tensor(sa / (sa * sw * math.sqrt(h)))
        sd[f"{pre}.self_attn.{name}.b"] = torch.tensor(0.05)
    sd[f"{pre}.self_attn.qk_bmm.a"] = torch.tensor(1.5 / (sa * sa * math.sqrt(h // heads)))
    sd[f"{pre}.self_attn.pv_bmm.a"] = torch.tensor(0.05)
    sd[f"{pre}.self_attn.out_proj.weight"] = s8(h, h)
    sd[f"{pre}.self_attn.out_proj.bias"] = torch.randn((1, h), generator=g) * 0.02
    sd[f"{pre}.self_attn.out_proj.a"] = torch.tensor(0.3 / (10.0 * sw * math.sqrt(h)))
    sd[f"{pre}.fc1.weight"] = s8(ffn, h)
    sd[f"{pre}.fc1.bias"] = s8(1, ffn)
    sd[f"{pre}.fc1.a"] = torch.tensor(40.0 / (sa * sw * math.sqrt(h)))
    sd[f"{pre}.fc1.b"] = torch.tensor(0.05)
    sd[f"{pre}.fc2.weight"] = s8(h, ffn)
    sd[f"{pre}.fc2.bias"] = torch.randn((1, h), generator=g) * 0.02
    sd[f"{pre}.fc2.a"] = torch.tensor(0.3 / (25.0 * sw * math.sqrt(ffn)))
    for ln in ("self_attn_layer_norm", "final_layer_norm"):
        sd[f"{pre}.{ln}.weight"] = torch.randn(h, generator=g) * (0.1 * sa) + sa
        sd[f"{pre}.{ln}.bias"] = torch.randn(h, generator=g) * (0.1 * sa)
    return sd, pre, heads


def opt_cpu_sample(arch, batch, seq, tokens=None):
    """Bounded CPU sample: ONE decoder layer at the full dimensions of `arch` on one whole sequence
    (`tokens` = min(seq, 512) tokens, so the host is compute bound rather than streaming the layer's
    weights for a few rows), evaluated by the oracle; the rate is extrapolated to the whole model as
    tokens / (layer time x layers) and labelled as such."""
    from oracle import opt_model as OM
    from oracle import w8a8 as O
    tokens = tokens or min(seq, 512)
    layers = OPT_DIMS[arch][1]
    sd, prefix, heads = reference_layer_state(arch)
    g = torch.Generator().manual_seed(1)
    hidden = torch.randn((1, tokens, OPT_DIMS[arch][0]), generator=g)
    mask = O.causal_mask(1, tokens, tokens)

    def run():
        return OM.decoder_layer(sd, prefix, hidden, mask, heads)
    units = tokens / float(layers)  # tokens per (layer-time x layers)
    return run, units, (f"one {arch} decoder layer at full dimensions on one {tokens}-token sequence, "
                        f"extrapolated x{layers} layers (embeddings and lm_head not included)"), O.num_threads()


# ------------------------------------------------------------- op-level workloads (HBM bound)
def _event_time(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


class RowKernelWorkload:
    """LayerNormQ, dq_add_layernorm_q and softmax_q at the shapes of the OPT-13B layer config
    ([4,512,5120]) and of the OPT-175B config ([16,1024,12288]); several buffers are rotated so that
    no launch finds its input in L2.  value = GB/s of the dq_add_layernorm_q kernel at the large shape."""
    name = "row_kernels_layernormq_dq_add_ln_q_softmax_q"
    metric = "dq_add_layernorm_q_gbytes_per_s"
    unit = "GB/s"
    dtype = "f32"
    scaling = "weak"
    launches_per_step = 1

    def __init__(self, device):
        from torch_int import _CUDA as C
        self.C, self.device = C, device
        self.h2d = self.d2h = 0
        self.cases = {}
        rot = 3
        rows, h = 16 * 1024, 12288
        self.acc = [torch.randint(-200000, 200000, (rows, h), dtype=torch.int32, device=device) for _ in range(rot)]
        self.res = [torch.randn((rows, h), device=device) for _ in range(rot)]
        self.gamma = torch.rand(h, device=device) * 20 + 10
        self.beta = torch.randn(h, device=device)
        self.i = 0
        self.bytes_per_step = rows * h * 13.0

    def step(self):
        self.i = (self.i + 1) % len(self.acc)
        return self.C.dq_add_layernorm_q(self.acc[self.i], 1e-5, self.res[self.i], self.gamma, self.beta, 1e-5)

    step_e2e = step

    def units(self, n_gpus):
        return self.bytes_per_step * n_gpus / 1e9

    def measure_cases(self, peaks):
        C, dev = self.C, self.device
        out = {}
        for label, (rows, h) in {"4x512x5120": (2048, 5120), "16x1024x12288": (16384, 12288)}.items():
            rot = 4 if rows * h < 5e7 else 3
            xs = [torch.randn((rows, h), device=dev) for _ in range(rot)]
            accs = [torch.randint(-200000, 200000, (rows, h), dtype=torch.int32, device=dev) for _ in range(rot)]
            g, b = torch.rand(h, device=dev) * 20 + 10, torch.randn(h, device=dev)
            k = [0]

            def ln():
                k[0] = (k[0] + 1) % rot
                C.layernorm_q(xs[k[0]], g, b, 1e-5)

            def dq():
                k[0] = (k[0] + 1) % rot
                C.dq_add_layernorm_q(accs[k[0]], 1e-5, xs[k[0]], g, b, 1e-5)
            for name, fn, bpe in (("layernorm_q", ln, 5.0), ("dq_add_layernorm_q", dq, 13.0)):
                ms = _event_time(fn, 50)
                gbs = rows * h * bpe / (ms * 1e-3) / 1e9
                out[f"{name} {label}"] = {"ms": round(ms, 4), "GB/s": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)}
            del xs, accs
        for label, (bh, t, s) in {"4x40 heads, S=512": (160, 512, 512), "4x40 heads, S=2048": (160, 2048, 2048)}.items():
            sc = [torch.randn((bh, t, s), device=dev) * 2 for _ in range(2)]
            k = [0]

            def sm():
                k[0] ^= 1
                C.softmax_q(sc[k[0]], None, 40, causal=0)
            ms = _event_time(sm, 20)
            # causal: on average half of each row is read; all of it is written
            gbs = bh * t * s * (4.0 * 0.5 + 1.0) / (ms * 1e-3) / 1e9
            out[f"softmax_q causal {label}"] = {"ms": round(ms, 4), "GB/s (algorithmic: half read + all written)": round(gbs, 1),
                                                "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)}
            del sc
        return out

    def config(self, n_gpus):
        return {"workload": self.name, "rows": 16384, "H": 12288, "bytes_per_element": 13,
                "l2": "three rotating input sets of 1.6 GB each: no launch finds its input in L2"}

    def roofline(self, ms, peaks):
        gbs = self.bytes_per_step / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(gbs / peaks["hbm_gbs"], 4), "traffic": None,
                "kernel": "dq_add_layernorm_q_kernel<float, 256, 12> at [16384, 12288] (13 B/element)",
                "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})",
                "cases": self.measure_cases(peaks)}

    def cpu_sample(self):
        from oracle import w8a8 as O
        rows, h = 512, 12288
        acc = torch.randint(-200000, 200000, (rows, h), dtype=torch.int32)
        res, g, b = torch.randn(rows, h), torch.rand(h) * 20 + 10, torch.randn(h)

        def run():
            return O.dq_add_layernorm_q(acc, 1e-5, res, g, b, 1e-5)
        return run, rows * h * 13.0 / 1e9, f"{rows} of 16384 rows (the reference's dq_add_layernorm_q_py on CPU)", torch.get_num_threads()


class BmmWorkload:
    """The attention products at batch*heads = 4*40, head_dim 128, seq 128/512/2048: Q.K^T -> fp32 and
    P.V -> int8.  value = GB/s (algorithmic bytes) of Q.K^T at S = 2048, which is HBM-write bound."""
    name = "attention_bmm_sweep_bh160_d128"
    metric = "bmm_s8t_s8n_f32t_gbytes_per_s"
    unit = "GB/s"
    dtype = "int8"
    scaling = "weak"
    launches_per_step = 1

    def __init__(self, device):
        from torch_int import _CUDA as C
        self.C, self.device = C, device
        self.h2d = self.d2h = 0
        bh, s, d = 160, 2048, 128
        self.q = torch.randint(-127, 128, (bh, s, d), dtype=torch.int8, device=device)
        self.k = torch.randint(-127, 128, (bh, s, d), dtype=torch.int8, device=device)
        self.bytes_per_step = bh * (2 * s * d + 4.0 * s * s)

    def step(self):
        return self.C.bmm_s8t_s8n_f32t(self.q, self.k, 1.0 / 127 ** 2)

    step_e2e = step

    def units(self, n_gpus):
        return self.bytes_per_step * n_gpus / 1e9

    def config(self, n_gpus):
        return {"workload": self.name, "batch_heads": 160, "head_dim": 128, "seq": 2048,
                "l2": "the 2.7 GB fp32 output exceeds L2"}

    def roofline(self, ms, peaks):
        C, dev = self.C, self.device
        cases = {}
        bh, d = 160, 128
        for s in (128, 512, 2048):
            q = torch.randint(-127, 128, (bh, s, d), dtype=torch.int8, device=dev)
            k = torch.randint(-127, 128, (bh, s, d), dtype=torch.int8, device=dev)
            p = torch.randint(-127, 128, (bh, s, s), dtype=torch.int8, device=dev)
            vt = torch.randint(-127, 128, (bh, d, s), dtype=torch.int8, device=dev)
            t1 = _event_time(lambda: C.bmm_s8t_s8n_f32t(q, k, 1.0 / 127 ** 2), 20)
            t2 = _event_time(lambda: C.bmm_s8t_s8n_s8t(p, vt, 0.01), 20)
            b1, b2 = bh * (2 * s * d + 4.0 * s * s), bh * (s * s + 2.0 * s * d)
            ops = 2.0 * bh * s * s * d
            cases[f"S={s}"] = {"qk_f32t_ms": round(t1, 4), "qk_GB/s": round(b1 / t1 / 1e6, 1), "qk_TOP/s": round(ops / t1 / 1e9, 1),
                               "pv_s8t_ms": round(t2, 4), "pv_GB/s": round(b2 / t2 / 1e6, 1), "pv_TOP/s": round(ops / t2 / 1e9, 1)}
            # the whole causal attention core of one layer: scores -> softmax -> context (three kernels) ...
            def three():
                sc = C.bmm_s8t_s8n_f32t(q, k, 1.0 / 127 ** 2)
                return C.bmm_s8t_s8n_s8t(C.softmax_q(sc, None, 40, causal=0), vt, 0.01)
            cases[f"S={s}"]["core_3_kernels_ms"] = round(_event_time(three, 10), 4)
            # ... and as the one fused kernel (scores and probabilities never leave the SM)
            out = torch.empty((4, s, 40 * d), dtype=torch.int8, device=dev)
            q4 = q.view(4, 40, s, d).transpose(1, 2).contiguous()      # [B, S, H*D] rows, heads side by side
            k4 = k.view(4, 40, s, d).transpose(1, 2).contiguous()
            cases[f"S={s}"]["core_fused_ms"] = round(_event_time(lambda: C.attention_prefill(
                q4, k4, vt, out, batch=4, heads=40, head_dim=d, tgt_len=s, src_len=s, ld_q=40 * d,
                q_batch_stride=s * 40 * d, ld_k=40 * d, k_batch_stride=s * 40 * d, ld_vt=s,
                alpha_qk=1.0 / 127 ** 2, alpha_pv=0.01), 10), 4)
        gbs = self.bytes_per_step / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(gbs / peaks["hbm_gbs"], 4), "traffic": None,
                "kernel": "gemm_i8_kernel<256, EPI_F32_ALPHA, PAIR> on [160, 2048, 128] x [160, 2048, 128]^T",
                "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peaks['source']})", "cases": cases}

    def cpu_sample(self):
        from oracle import w8a8 as O
        g = torch.Generator().manual_seed(0)
        q = torch.randint(-127, 128, (4, 2048, 128), generator=g, dtype=torch.int8)
        k = torch.randint(-127, 128, (4, 2048, 128), generator=g, dtype=torch.int8)

        def run():
            return O.bmm_s8t_s8n_f32t(q, k, 1.0 / 127 ** 2)
        return run, 4 * (2 * 2048 * 128 + 4.0 * 2048 * 2048) / 1e9, "4 of the 160 (batch, head) products at S = 2048", O.num_threads()


def time_steps(fn, steps, warmup, world):
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def cpu_baseline(wl, min_seconds=10.0, max_reps=50):
    run, units, sample, cores = wl.cpu_sample()
    run()  # warm-up (page in, spin up the thread pool)
    t0 = time.perf_counter()
    reps = 0
    while True:
        run()
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or reps >= max_reps:
            break
    return {"value": round(units * reps / dt, 4), "unit": wl.unit, "cores": cores, "kind": "port",
            "sample": f"{sample}; {reps} repetitions in {dt:.1f} s"}


def pick_workload(name, world):
    if name in (None, "auto"):
        name = "opt30b" if world == 1 else "opt175b"
    if name in ("gemm", "norm", "bmm") or name in OPT_WORKLOADS:
        return name
    raise SystemExit(f"unknown workload {name}")


def run_reference(args, world, rank):
    """CPU arm: the reference semantics on the host cores (the oracle's C port; the reference
    itself has no CPU implementation of its GEMM/BMM path and cannot be built without CUTLASS).
    Loads neither this repository's package nor its CUDA library."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    key = pick_workload(args.workload, world)
    if key == "gemm":
        wl = GemmWorkload.__new__(GemmWorkload)
        m, n, k = HG
        g = torch.Generator().manual_seed(0)
        wl.x_host = torch.randint(-127, 128, (128, k), generator=g, dtype=torch.int8)
        g1 = torch.Generator().manual_seed(1)
        wl.w = torch.randint(-127, 128, (n, k), generator=g1, dtype=torch.int8)
        wl.b = torch.randint(-127, 128, (n,), generator=g1, dtype=torch.int8)
        wl.alpha, wl.beta = 1e-4, 0.01
        run, units, sample, cores = wl.cpu_sample()
        metric, unit, dtype, scaling = GemmWorkload.metric, GemmWorkload.unit, GemmWorkload.dtype, GemmWorkload.scaling
        config = GemmWorkload.config(wl, world)
    elif key in ("norm", "bmm"):
        WL = RowKernelWorkload if key == "norm" else BmmWorkload
        run, units, sample, cores = WL.cpu_sample(None)
        metric, unit, dtype, scaling = WL.metric, WL.unit, WL.dtype, WL.scaling
        config = WL.config(WL.__new__(WL), world)
    else:
        arch, batch, seq, _ = OPT_WORKLOADS[key]
        tokens = min(seq, 512)
        while True:
            run, units, sample, cores = opt_cpu_sample(arch, batch, seq, tokens)
            t0 = time.perf_counter()
            run()
            first = time.perf_counter() - t0
            # keep the whole --steps/--warmup run within a few minutes: halve the sample if it would not fit
            if first * (min(args.steps, 20) + 2) <= 240.0 or tokens <= 64:
                break
            tokens //= 2
        metric, unit, dtype, scaling = OptWorkload.metric, OptWorkload.unit, OptWorkload.dtype, OptWorkload.scaling
        config = opt_config_dict(key, world)
    for _ in range(max(1, min(args.warmup, 2))):
        run()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    value = units * steps / dt
    extra = {}
    if key == "gemm":
        extra = reference_cuda_kernel_rate()
    line = {"impl": "reference", "metric": metric, "value": round(value, 4), "unit": unit,
            "n_gpus": world, "steps": steps, "warmup": args.warmup,
            "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": dtype, "data": "synthetic (seeded random int8 weights and inputs)",
            "config": config,
            "cpu_baseline": {"value": round(value, 4), "unit": unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 4), "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    line.update(extra)
    print(json.dumps(line), flush=True)


def reference_cuda_kernel_rate():
    """Extra key of the CPU arm's gemm line, when a GPU and the reference's own extension are there
    (oracle/_ref/ref_torch_int.so: its CUTLASS 2.x Sm80 mma.sync kernels, built from the reference's sources and
    translated by the driver for this GPU): TOP/s of the reference's linear_a8_w8_b8_o8 on the headline shape.
    Informational - the arm's `value` stays the host-core figure."""
    try:
        if not torch.cuda.is_available():
            return {}
        from oracle import build_ref_gemm
        ref = build_ref_gemm.load()
        if ref is None:
            return {}
        m, n, k = HG
        dev = torch.device("cuda", 0)
        x = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 128, (n,), dtype=torch.int8, device=dev)
        ms = _event_time(lambda: ref.linear_a8_w8_b8_o8(x, w, b, 1e-4, 0.01), 20)
        return {"reference_cuda_kernel": {"op": "linear_a8_w8_b8_o8 (CUTLASS 2.x Sm80 mma.sync, PTX translated for this GPU)",
                                          "shape": [m, n, k], "ms": round(ms, 4),
                                          "tops": round(2.0 * m * n * k / (ms * 1e-3) / 1e12, 1)}}
    except Exception as exc:  # noqa: BLE001 - an optional extra must not break the arm
        return {"reference_cuda_kernel": {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}}


def profile_one_step(wl, region):
    """One step of the OPT workload inside the CUDA profiler range (everything before it is warm-up)."""
    model = wl.model
    for _ in range(2):
        wl.step()
    if region == "prefill":
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        wl.step()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    else:
        cache = model.new_cache(wl.batch, wl.seq + 16)
        out = model(wl.ids, past_key_values=cache, use_cache=True, last_token_only=True)
        nxt = out.logits[:, -1, :].argmax(dim=-1, keepdim=True)
        for _ in range(3):
            nxt = model.decode_step(nxt, cache).argmax(dim=-1, keepdim=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        nxt = model.decode_step(nxt, cache).argmax(dim=-1, keepdim=True)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    print(json.dumps({"profiled": region, "workload": wl.name}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode-rate measurement of the OPT workloads")
    ap.add_argument("--trace", default=None, metavar="DIR",
                    help="tensor-parallel OPT workloads: after the measurement run one more step with CUDA events "
                         "around every compute phase and exchange stage, write DIR/tp_trace_rank<r>.json (Chrome "
                         "trace format) and add the per-stream busy times to the JSON line")
    ap.add_argument("--profile", action="store_true",
                    help="kernel-only run for ncu: no end-to-end leg, no CPU baseline")
    ap.add_argument("--shape", default=None, metavar="M,N,K",
                    help="gemm workload: another problem size than the headline one (for profiler captures of the "
                         "models' per-layer GEMMs; the line then names that shape)")
    ap.add_argument("--profile-region", default=None, choices=["prefill", "decode"],
                    help="OPT workloads, one GPU: after warm-up, run ONE prefill step or ONE eager decode step between "
                         "cudaProfilerStart/Stop and exit (for `ncu --profile-from-start off`: the launch list of a step)")
    args = ap.parse_args()
    world, rank, local = dist_env()
    key = pick_workload(args.workload, world)
    if args.steps is None:
        args.steps = {"gemm": 1000, "norm": 200, "bmm": 100}.get(key, 10)
    if args.warmup is None:
        args.warmup = 5 if key in ("gemm", "norm", "bmm") else 3
    if args.impl == "reference":
        run_reference(args, world, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    dog = Watchdog(rank)
    deadline = int(os.environ.get("TI_BENCH_DEADLINE_S", "600"))
    dog.arm(deadline, "setup and prefill measurement")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import datetime
        import torch.distributed as dist
        # a collective that does not finish within this limit aborts the rank: well below the
        # deadline above, so that a hang is reported by the rank that saw it
        dist.init_process_group("nccl", device_id=device,
                                timeout=datetime.timedelta(seconds=int(os.environ.get("TI_BENCH_NCCL_TIMEOUT_S", "120"))))
        progress("process group initialised")
    if key == "gemm":
        if args.shape:
            global HG
            HG = tuple(int(v) for v in args.shape.split(","))
            GemmWorkload.name = "w8a8_gemm_%dx%dx%d_int8out" % HG
        wl = GemmWorkload(device)
    elif key == "norm":
        wl = RowKernelWorkload(device)
    elif key == "bmm":
        wl = BmmWorkload(device)
    else:
        wl = OptWorkload(device, key, world, rank)
    progress(f"workload {key} built, first step done")
    peaks = measured_peaks()
    from torch_int import _CUDA as C
    if args.profile_region and key in OPT_WORKLOADS:
        profile_one_step(wl, args.profile_region)
        dog.disarm()
        return

    def agreed_max(value):
        """Maximum of an integer over the ranks: every rank then takes the same decision."""
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([int(value)], dtype=torch.int32, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            value = int(t.item())
        return int(value)

    def agreed_status():
        return agreed_max(C.device_status(reset=True))

    if key in OPT_WORKLOADS and world > 1:
        st = agreed_status()
        peer = agreed_max(1 if wl.tp.use_peer_memory else 0)   # a per-rank flag: agree on it before branching
        if st != 0 and peer:
            # the first step (run while the workload was built) hit a bounded-wait time limit in the
            # peer-memory exchange: all ranks use NCCL collectives for the measurement instead
            progress(f"first step reported status {st}: switching every rank to the NCCL exchange")
            wl.tp.use_peer_memory = False
            wl.step()
            st = agreed_status()
        assert st == 0, f"a kernel reported wait timeout {st}"

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = time_steps(wl.step, args.steps, args.warmup, world)
    clocks = sampler.stop() if sampler else None
    progress(f"prefill timed: {ms:.3f} ms/step")
    ms_e2e = ms if args.profile else time_steps(wl.step_e2e, args.steps, args.warmup, world)
    progress(f"end-to-end timed: {ms_e2e:.3f} ms/step")
    status = agreed_status()
    assert status == 0, f"a kernel reported wait timeout {status}"
    agree = None
    if key in OPT_WORKLOADS and world > 1 and not args.profile:
        agree = bool(agreed_max(0 if wl.ranks_agree() else 1) == 0)
    line = None
    if rank == 0:
        units = wl.units(world)
        line = {"metric": wl.metric, "value": round(units / (ms * 1e-3), 2), "unit": wl.unit, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
                "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype,
                "data": "synthetic (seeded random int8 weights and inputs)", "config": wl.config(world),
                "e2e": {"value": round(units / (ms_e2e * 1e-3), 2), "unit": wl.unit,
                        "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                        "ms_per_step": round(ms_e2e, 4)},
                "gpu_launches": wl.launches_per_step * args.steps, "clocks": clocks}
        if key in OPT_WORKLOADS:
            line["tp_exchange"] = wl.exchange()
        if agree is not None:
            line["tp_ranks_agree"] = agree
    # From here on a failure must not lose the measurement: the watchdog prints `line` as it stands.
    dog.line, dog.salvageable = line, True
    leg_deadline = int(os.environ.get("TI_BENCH_LEG_DEADLINE_S", "100"))
    extra = {}
    if key in OPT_WORKLOADS and not args.profile and not args.no_decode:
        dog.arm(leg_deadline, "decode")
        try:
            extra.update(wl.decode_rate())
            st = agreed_status()
            if st != 0:
                extra["decode_error"] = f"a kernel reported wait timeout {st}"
        except Exception as exc:  # noqa: BLE001 - reported in the line; the prefill measurement stands
            extra["decode_error"] = f"{type(exc).__name__}: {exc}"
        progress("decode leg done")
    if args.trace and key in OPT_WORKLOADS and world > 1:
        dog.arm(leg_deadline, "trace")
        from torch_int.models.tensor_parallel import StreamTrace
        wl.tp.trace = StreamTrace()
        wl.step()
        torch.cuda.synchronize()
        trace, wl.tp.trace = wl.tp.trace, None
        os.makedirs(args.trace, exist_ok=True)
        trace.dump(os.path.join(args.trace, f"tp_trace_rank{rank}.json"), pid=rank)
        extra["tp_trace"] = {row: {"busy_ms": round(v["busy_us"] / 1e3, 2),
                                   "extent_ms": round((v["last_us"] - v["first_us"]) / 1e3, 2),
                                   "by_name_ms": {k: round(t / 1e3, 2) for k, t in v["by_name"].items()}}
                             for row, v in trace.summary().items()}
        progress("trace leg done")
    if rank == 0:
        dog.arm(leg_deadline + 60, "roofline and CPU baseline")
        line.update(extra)
        line["roofline"] = wl.roofline(ms, peaks)
        if world == 1 and not args.no_cpu_baseline and not args.profile:
            line["cpu_baseline"] = cpu_baseline(wl)
        dog.disarm()
        print(json.dumps(line), flush=True)
    dog.disarm()
    progress("line printed" if rank == 0 else "done")
    if world > 1:
        import torch.distributed as dist
        dog.arm(60, "teardown")
        dist.destroy_process_group()
        dog.disarm()


if __name__ == "__main__":
    main()
